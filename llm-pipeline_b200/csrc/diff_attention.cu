// Differential attention: every query head has two score maps (two queries of `d` entries against two keys of `d`
// entries of its key/value head), each with a softmax of its own over the same values of `dv` entries; a head's
// output is a1 - lambda a2, divided by its root mean square over the dv entries and scaled by a constant.
//
// A token's cache row, per key/value head, is [key of map 1 | key of map 2 | value] = 2 d + dv entries; pages are
// [page, kv head, token in page, 2 d + dv].
//
//   diff_qkv_post:  per token, on the product [q | k | v] = [H 2 d | G 2 d | G dv]: RMS norm with a weight over every
//                   run of d entries of q and k (one weight for all of q, one for all of k), rotation of the first
//                   `rot` entries of each run (entry i with entry i + rot / 2), q back in place, k and v to the
//                   token's place in the pages.
//   diff_attention_kernel: the general kernel (float32 or bfloat16, any sizes, any mix of portions, sliding window):
//                   a warp per (token, query head), key tiles of 32 aligned to key 0, so a row's operations do not
//                   depend on the step. Scores, both softmaxes, the difference and its norm are float32.
#include "common.cuh"

#define DA_KEYS 32
#define DA_WARPS 8
#define DA_POST_THREADS 256
#define DA_MAX_D 256

// One block per token. The whole row [q | k | v] goes to shared memory in one sweep of 16-byte loads (all in flight at
// once). Norm weight and rotation are folded into two coefficient vectors per token, for q and for k:
// out[i] = rstd (x[i] A[i] + x[partner(i)] B[i]) with A = w cos, B = -/+ w[partner] sin inside the rotated part and
// A = w, B = 0 outside it. Then a warp owns a run of d entries at a time: sum of squares, the two products per entry, and
// the store to the run's place (q back into the row, k into the token's cache rows), two entries a lane where the sizes
// are even. v is copied to the cache rows as it is.
template <typename T> struct PostPair;
template <> struct PostPair<float> { typedef float2 type; static __device__ __forceinline__ float2 make(float a, float b) { return make_float2(a, b); } };
template <> struct PostPair<bf16> { typedef __nv_bfloat162 type; static __device__ __forceinline__ __nv_bfloat162 make(float a, float b) { return __floats2bfloat162_rn(a, b); } };

template <typename T, bool VEC>
__global__ void __launch_bounds__(DA_POST_THREADS)
diff_qkv_post_kernel(T* __restrict__ qkv, long ld, int H, int G, int d, int dv, const void* __restrict__ qw, const void* __restrict__ kw,
                     int w_bf16, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                     const int* __restrict__ slots, T* __restrict__ pages, int page_size) {
    extern __shared__ __align__(16) unsigned char post_raw[];
    const int units = 2 * H + 2 * G, q_units = 2 * H;
    const int qk = units * d, width = qk + G * dv;
    const int half = rot / 2;
    float* coef = reinterpret_cast<float*>(post_raw);        // [2][2][d]: A and B for q, then for k
    T* vals = reinterpret_cast<T*>(post_raw + (((size_t)(4 * d) * sizeof(float) + 15) / 16) * 16);   // [width]: the row as stored
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    pdl_wait();
    pdl_trigger();
    T* row = qkv + (size_t)n * ld;
    for (int e = threadIdx.x; e < 2 * d; e += blockDim.x) {
        const int which = e >= d, i = which ? e - d : e;
        const void* w = which ? kw : qw;
        float a = load_as_float(w, w_bf16, i), b = 0.f;
        if (i < half) {
            const float c = cos_t[(size_t)n * half + i], sv = sin_t[(size_t)n * half + i];
            b = -load_as_float(w, w_bf16, i + half) * sv;
            a *= c;
        } else if (i < rot) {
            const float c = cos_t[(size_t)n * half + i - half], sv = sin_t[(size_t)n * half + i - half];
            b = load_as_float(w, w_bf16, i - half) * sv;
            a *= c;
        }
        coef[which * 2 * d + i] = a;
        coef[which * 2 * d + d + i] = b;
    }
    const int slot = slots ? slots[n] : -1;
    const int rs = 2 * d + dv;
    T* page_row = nullptr;                                   // the token's row of key/value head 0
    if (pages && slot >= 0)
        page_row = pages + (((size_t)(slot / page_size) * G) * page_size + slot % page_size) * rs;
    const size_t head_step = (size_t)page_size * rs;         // from one key/value head's row to the next one's
    const int live = page_row ? width : q_units * d;         // without a cache row keys and values are not needed
    if (VEC) {
        constexpr int PER = 16 / sizeof(T);
        const uint4* src = reinterpret_cast<const uint4*>(row);
        uint4* dst = reinterpret_cast<uint4*>(vals);
        for (int e = threadIdx.x; e < live / PER; e += blockDim.x) dst[e] = src[e];
    } else {
        for (int e = threadIdx.x; e < live; e += blockDim.x) vals[e] = row[e];
    }
    __syncthreads();
    if (page_row) {                                          // the values pass as they are
        const T* v = vals + qk;
        if (VEC) {
            constexpr int PER = 16 / sizeof(T);
            const int per_head = dv / PER;
            for (int e = threadIdx.x; e < G * per_head; e += blockDim.x) {
                const int g = e / per_head, c = e - g * per_head;
                reinterpret_cast<uint4*>(page_row + (size_t)g * head_step + 2 * d)[c] = reinterpret_cast<const uint4*>(v + (size_t)g * dv)[c];
            }
        } else {
            for (int e = threadIdx.x; e < G * dv; e += blockDim.x) {
                const int g = e / dv, c = e - g * dv;
                page_row[(size_t)g * head_step + 2 * d + c] = v[e];
            }
        }
    }
    const int live_units = page_row ? units : q_units;
    for (int u = warp; u < live_units; u += nwarps) {
        const T* x = vals + u * d;
        const bool is_key = u >= q_units;
        const float* A = coef + (is_key ? 2 * d : 0);
        const float* B = A + d;
        float ss = 0.f;
        for (int i = lane; i < d; i += 32) {
            const float v = to_float(x[i]);
            ss = fmaf(v, v, ss);
        }
        const float r = rsqrtf(warp_sum(ss) / (float)d + eps);
        T* dst = row + (size_t)u * d;
        if (is_key) {
            const int ku = u - q_units;                      // key/value head ku / 2, map ku % 2
            dst = page_row + (size_t)(ku >> 1) * head_step + (size_t)(ku & 1) * d;
        }
        auto entry = [&](int i) {
            const int partner = i < half ? i + half : (i < rot ? i - half : i);
            return r * fmaf(to_float(x[i]), A[i], to_float(x[partner]) * B[i]);
        };
        if (VEC) {                                           // d is even and every run starts on a 4-byte boundary
            for (int i = 2 * lane; i < d; i += 64)
                *reinterpret_cast<typename PostPair<T>::type*>(dst + i) = PostPair<T>::make(entry(i), entry(i + 1));
        } else {
            for (int i = lane; i < d; i += 32) dst[i] = from_float<T>(entry(i));
        }
    }
}

LLMP_API int llmp_diff_qkv_post(void* qkv, int dtype, long ld, int H, int G, int d, int dv, const void* q_weight, const void* k_weight,
                                int w_dtype, float eps, const float* cos_t, const float* sin_t, int rot, const int* slots, void* pages,
                                int page_size, int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && d > 0 && d <= DA_MAX_D && dv > 0 && rot >= 0 && rot <= d && rot % 2 == 0,
                 "diff_qkv_post: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d rotated=%d", H, G, d, dv, rot);
    LLMP_REQUIRE(rot == 0 || (cos_t && sin_t), "diff_qkv_post: a rotation needs its tables");
    LLMP_REQUIRE(!pages || (slots && page_size > 0), "diff_qkv_post: pages need slots and a page size");
    const size_t elem = dtype == LLMP_F32 ? 4 : 2;
    const size_t width = (size_t)(2 * H + 2 * G) * d + (size_t)G * dv;
    const size_t smem = (((size_t)(4 * d) * sizeof(float) + 15) / 16) * 16 + width * elem + 16;
    LLMP_REQUIRE(smem <= 200 * 1024, "diff_qkv_post: %d heads of %d entries do not fit shared memory", H, d);
    // 16-byte pieces and pairs of entries: every run, row and cache row must start on such a boundary
    const int per = (int)(16 / elem);
    const bool vec = d % per == 0 && dv % per == 0 && ld % per == 0 && ((size_t)qkv % 16) == 0 && ((size_t)pages % 16) == 0;
    cudaError_t e;
#define LLMP_POST(T, V)                                                                                                              \
    do {                                                                                                                             \
        LLMP_ALLOW_SMEM((diff_qkv_post_kernel<T, V>), smem);                                                                         \
        e = llmp_launch_dependent(diff_qkv_post_kernel<T, V>, dim3(N), dim3(DA_POST_THREADS), smem, stream, (T*)qkv, ld, H, G, d, dv, \
                                  q_weight, k_weight, (int)(w_dtype == LLMP_BF16), eps, cos_t, sin_t, rot, slots, (T*)pages, page_size); \
    } while (0)
    if (dtype == LLMP_F32) {
        if (vec) LLMP_POST(float, true); else LLMP_POST(float, false);
    } else {
        if (vec) LLMP_POST(bf16, true); else LLMP_POST(bf16, false);
    }
#undef LLMP_POST
    LLMP_REQUIRE(e == cudaSuccess, "diff_qkv_post: %s", cudaGetErrorString(e));
    return llmp_check_launch("diff_qkv_post");
}

struct DiffArgs {
    const void* q; long q_t;                 // [token, head, map, d]: stride of a token in elements
    const void* pages;                       // [page, kv head, token in page, 2 d + dv]
    const int* tables; int width;            // [requests, width]
    const int* token_request; const int* positions;
    void* out; long o_t;                     // [token, head, dv]
    int H, G, d, dv, page_size, window;
    float scale, lambda, eps, out_scale;
};

template <typename T, int NO>
__global__ void __launch_bounds__(DA_WARPS * 32) diff_attention_kernel(const DiffArgs a) {
    extern __shared__ float smem[];
    const int nw = blockDim.x >> 5;
    const int rs = 2 * a.d + a.dv;
    const int ks = rs | 1;                                   // odd row stride: the lanes of a warp hit different banks
    float* Ks = smem;                                        // [DA_KEYS][ks]
    float* qs = Ks + DA_KEYS * ks;                           // [nw][2 d]
    float* ps = qs + nw * 2 * a.d;                           // [nw][2][DA_KEYS]
    const int n = blockIdx.x, g = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hpg = a.H / a.G;
    const int hi = blockIdx.z * nw + warp;
    const bool active = hi < hpg;
    const int h = g * hpg + hi;
    const int pos = a.positions[n];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int* table = a.tables + (size_t)a.token_request[n] * a.width;
    const T* pages = reinterpret_cast<const T*>(a.pages);
    float* qw = qs + warp * 2 * a.d;
    if (active) {
        const T* q = reinterpret_cast<const T*>(a.q) + (size_t)n * a.q_t + (size_t)h * 2 * a.d;
        for (int i = lane; i < 2 * a.d; i += 32) qw[i] = to_float(q[i]) * a.scale;
    }
    float o1[NO], o2[NO];
#pragma unroll
    for (int i = 0; i < NO; ++i) o1[i] = o2[i] = 0.f;
    float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.f, l2 = 0.f;
    float* p1 = ps + warp * 2 * DA_KEYS;
    float* p2 = p1 + DA_KEYS;
    for (int k0 = (lo / DA_KEYS) * DA_KEYS; k0 <= pos; k0 += DA_KEYS) {
        __syncthreads();
        for (int j = warp; j < DA_KEYS; j += nw) {           // a warp copies a key's row
            const int key = k0 + j;
            int page = -1;
            if (key >= lo && key <= pos) page = table[key / a.page_size];
            if (page >= 0) {
                const T* row = pages + (((size_t)page * a.G + g) * a.page_size + key % a.page_size) * rs;
                for (int i = lane; i < rs; i += 32) Ks[j * ks + i] = to_float(row[i]);
            } else {
                for (int i = lane; i < rs; i += 32) Ks[j * ks + i] = 0.f;
            }
        }
        __syncthreads();
        if (!active) continue;
        const int key = k0 + lane;
        const bool valid = key >= lo && key <= pos;
        const float* kr = Ks + lane * ks;
        float s1 = 0.f, s2 = 0.f;
        for (int i = 0; i < a.d; ++i) {
            s1 = fmaf(qw[i], kr[i], s1);
            s2 = fmaf(qw[a.d + i], kr[a.d + i], s2);
        }
        s1 = valid ? s1 : -INFINITY;
        s2 = valid ? s2 : -INFINITY;
        // every tile between the one that holds `lo` and the one that holds `pos` has a visible key: the maxima are finite
        const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
        const float e1 = valid ? expf(s1 - n1) : 0.f, e2 = valid ? expf(s2 - n2) : 0.f;
        const float al1 = expf(m1 - n1), al2 = expf(m2 - n2);       // 0 at the first tile
        l1 = l1 * al1 + warp_sum(e1);
        l2 = l2 * al2 + warp_sum(e2);
        m1 = n1;
        m2 = n2;
        p1[lane] = e1;
        p2[lane] = e2;
        __syncwarp();
        const int j_lo = max(0, lo - k0), j_hi = min(DA_KEYS - 1, pos - k0);
#pragma unroll
        for (int i = 0; i < NO; ++i) {
            const int c = lane + 32 * i;
            if (c < a.dv) {
                float x1 = o1[i] * al1, x2 = o2[i] * al2;
                for (int j = j_lo; j <= j_hi; ++j) {
                    const float v = Ks[j * ks + 2 * a.d + c];
                    x1 = fmaf(p1[j], v, x1);
                    x2 = fmaf(p2[j], v, x2);
                }
                o1[i] = x1;
                o2[i] = x2;
            }
        }
        __syncwarp();
    }
    if (!active) return;
    const float i1 = 1.f / l1, i2 = a.lambda / l2;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NO; ++i) {
        const int c = lane + 32 * i;
        o1[i] = c < a.dv ? o1[i] * i1 - o2[i] * i2 : 0.f;
        ss += o1[i] * o1[i];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)a.dv + a.eps) * a.out_scale;
    T* dst = reinterpret_cast<T*>(a.out) + (size_t)n * a.o_t + (size_t)h * a.dv;
#pragma unroll
    for (int i = 0; i < NO; ++i) {
        const int c = lane + 32 * i;
        if (c < a.dv) dst[c] = from_float<T>(o1[i] * r);
    }
}

template <typename T>
static int launch_diff(const DiffArgs& a, int N, cudaStream_t stream) {
    const int hpg = a.H / a.G;
    const int nw = hpg < DA_WARPS ? hpg : DA_WARPS;
    const int rs = 2 * a.d + a.dv;
    const size_t smem = ((size_t)DA_KEYS * (rs | 1) + (size_t)nw * 2 * a.d + (size_t)nw * 2 * DA_KEYS) * sizeof(float);
    LLMP_REQUIRE(smem <= 220 * 1024, "diff_attention: rows of %d entries do not fit shared memory", rs);
    dim3 grid(N, a.G, (hpg + nw - 1) / nw);
#define LLMP_DA_LAUNCH(NO)                                                  \
    do {                                                                    \
        LLMP_ALLOW_SMEM((diff_attention_kernel<T, NO>), smem);              \
        diff_attention_kernel<T, NO><<<grid, nw * 32, smem, stream>>>(a);   \
    } while (0)
    if (a.dv <= 32) LLMP_DA_LAUNCH(1);
    else if (a.dv <= 64) LLMP_DA_LAUNCH(2);
    else if (a.dv <= 128) LLMP_DA_LAUNCH(4);
    else if (a.dv <= 256) LLMP_DA_LAUNCH(8);
    else LLMP_DA_LAUNCH(16);
#undef LLMP_DA_LAUNCH
    return llmp_check_launch("diff_attention");
}

LLMP_API int llmp_diff_attention(const void* q, long q_t, const void* pages, int dtype, const int* tables, int width,
                                 const int* token_request, const int* positions, void* out, long o_t, int N, int H, int G, int d,
                                 int dv, int page_size, int window, float scale, float lambda, float eps, float out_scale,
                                 cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0 && dv <= 512 && page_size > 0 && width > 0 && window >= 0,
                 "diff_attention: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d page=%d width=%d window=%d", H, G, d, dv, page_size,
                 width, window);
    LLMP_REQUIRE(G <= 65535 && H / G <= 65535 * DA_WARPS, "diff_attention: too many heads %d", H);
    DiffArgs a;
    a.q = q; a.q_t = q_t; a.pages = pages; a.tables = tables; a.width = width; a.token_request = token_request;
    a.positions = positions; a.out = out; a.o_t = o_t;
    a.H = H; a.G = G; a.d = d; a.dv = dv; a.page_size = page_size; a.window = window;
    a.scale = scale; a.lambda = lambda; a.eps = eps; a.out_scale = out_scale;
    return dtype == LLMP_F32 ? launch_diff<float>(a, N, stream) : launch_diff<bf16>(a, N, stream);
}
