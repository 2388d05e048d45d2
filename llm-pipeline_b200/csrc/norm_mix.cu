// Row kernels around the residual stream for blocks that norm a sublayer's output before it is added, and for models
// that mix the results of all earlier layers: embedding gather with its norm, the fused "norm the addend, add, keep
// the layer's result, mix over depth, norm for the next reader" kernel, the PolyNorm activation and the logit soft cap.
// Every statistic, the residual and the mixed sums are float32; a norm weight w is applied as (offset + w).
#include "common.cuh"

template <typename T> __device__ __forceinline__ float load_any(const void* p, size_t i) { return to_float(reinterpret_cast<const T*>(p)[i]); }

__device__ __forceinline__ float load_dt(const void* p, int is_bf16, size_t i) { return load_as_float(p, is_bf16, i); }

__device__ __forceinline__ void store_dt(void* p, int is_bf16, size_t i, float v) {
    if (is_bf16) reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(p)[i] = v;
}

// ------------------------------------------------------------------------------------------
// out[n, :] = rms_norm(table[ids[n], :]) * (offset + w), float32: the embedding with a norm of its own.
// ------------------------------------------------------------------------------------------
__global__ void embedding_norm_kernel(const int* __restrict__ ids, const void* __restrict__ table, int table_bf16,
                                      const void* __restrict__ w, int w_bf16, float offset, float eps, float* __restrict__ out,
                                      int H, int V) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    const int n = blockIdx.x;
    const int id = ids[n];
    const bool ok = id >= 0 && id < V;
    const size_t base = (size_t)(ok ? id : 0) * H;
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float x = ok ? load_dt(table, table_bf16, base + c) : 0.f;
        row[c] = x;
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        out[(size_t)n * H + c] = row[c] * r * (offset + load_dt(w, w_bf16, c));
}

LLMP_API int llmp_embedding_norm(const int* ids, const void* table, int table_dtype, const void* w, int w_dtype, float offset,
                                 float eps, float* out, int N, int H, int V, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && V > 0 && (size_t)H * 4 <= 200 * 1024, "embedding_norm: bad sizes H=%d V=%d", H, V);
    const size_t smem = (size_t)H * sizeof(float);
    LLMP_ALLOW_SMEM(embedding_norm_kernel, smem);
    embedding_norm_kernel<<<N, H >= 2048 ? 512 : 128, smem, stream>>>(ids, table, table_dtype == LLMP_BF16, w, w_dtype == LLMP_BF16,
                                                                      offset, eps, out, H, V);
    return llmp_check_launch("embedding_norm");
}

// ------------------------------------------------------------------------------------------
// The stream's norm kernel in its general form. For output row m (row r = rows ? rows[m] : m of the step):
//   y = delta[r]                                   (optional; float32 or bfloat16)
//   y = y * rsqrt(mean(y^2) + delta_eps) * (delta_offset + delta_w)       (if delta_w: the addend has a norm of its own)
//   x = residual[r] + y
//   if history:  history[index][r] = x;  x = sum_{j <= index} mix[j] * history[j][r]       (results of all layers so far)
//   residual[r] = x                               (only without `rows`)
//   out[m] = x * rsqrt(mean(x^2) + eps) * (offset + w)                     (if out)
// One block per row; the row stays in shared memory between the passes. history is [slots][T][H] float32.
// ------------------------------------------------------------------------------------------
struct NormMixArgs {
    float* residual;
    const void* delta; int delta_bf16;
    const void* delta_w; int delta_w_bf16; float delta_offset, delta_eps;
    float* history; long history_stride; const float* mix; int index;
    const void* w; int w_bf16; float offset, eps;
    void* out; int out_bf16;
    const int* rows; int H;
};

__global__ void add_norm_mix_kernel(const NormMixArgs a) {
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    const int H = a.H;
    float* xs = smem;
    const int m = blockIdx.x;
    const int r = a.rows ? a.rows[m] : m;
    const size_t base = (size_t)r * H;
    float scale_y = 1.f;
    if (a.delta && a.delta_w) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float y = load_dt(a.delta, a.delta_bf16, base + c);
            ss += y * y;
        }
        ss = block_sum(ss, scratch);
        scale_y = rsqrtf(ss / (float)H + a.delta_eps);
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x = a.residual[base + c];
        if (a.delta) {
            float y = load_dt(a.delta, a.delta_bf16, base + c);
            if (a.delta_w) y = y * scale_y * (a.delta_offset + load_dt(a.delta_w, a.delta_w_bf16, c));
            x += y;
        }
        if (a.history) {
            if (!a.rows) a.history[(size_t)a.index * a.history_stride + base + c] = x;
            float mixed = 0.f;
            for (int j = 0; j < a.index; ++j) mixed = fmaf(a.mix[j], a.history[(size_t)j * a.history_stride + base + c], mixed);
            x = fmaf(a.mix[a.index], x, mixed);
        }
        if (!a.rows && (a.delta || a.history)) a.residual[base + c] = x;
        xs[c] = x;
        ss += x * x;
    }
    if (!a.out) return;
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)H + a.eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x)
        store_dt(a.out, a.out_bf16, (size_t)m * H + c, xs[c] * rstd * (a.offset + load_dt(a.w, a.w_bf16, c)));
}

LLMP_API int llmp_add_norm_mix(float* residual, const void* delta, int delta_dtype, const void* delta_w, int delta_w_dtype,
                               float delta_offset, float delta_eps, float* history, long history_stride, const float* mix,
                               int index, const void* w, int w_dtype, float offset, float eps, void* out, int out_dtype,
                               const int* rows, int M, int H, cudaStream_t stream) {
    if (M <= 0) return 0;
    LLMP_REQUIRE(H > 0 && (size_t)H * 4 <= 200 * 1024, "add_norm_mix: bad width %d", H);
    LLMP_REQUIRE(!history || (mix && index >= 0), "add_norm_mix: a history needs mixing weights and an index");
    LLMP_REQUIRE(!out || w, "add_norm_mix: an output needs a norm weight");
    NormMixArgs a;
    a.residual = residual;
    a.delta = delta; a.delta_bf16 = delta_dtype == LLMP_BF16;
    a.delta_w = delta_w; a.delta_w_bf16 = delta_w_dtype == LLMP_BF16; a.delta_offset = delta_offset; a.delta_eps = delta_eps;
    a.history = history; a.history_stride = history_stride; a.mix = mix; a.index = index;
    a.w = w; a.w_bf16 = w_dtype == LLMP_BF16; a.offset = offset; a.eps = eps;
    a.out = out; a.out_bf16 = out_dtype == LLMP_BF16;
    a.rows = rows; a.H = H;
    const size_t smem = (size_t)H * sizeof(float);
    LLMP_ALLOW_SMEM(add_norm_mix_kernel, smem);
    // few rows (a decode step): as many threads as the row has pairs of entries, so that a thread's loads are few
    const int threads = (M <= 256 && H >= 512) ? (H >= 2048 ? 1024 : (H / 2 + 31) / 32 * 32) : (H >= 2048 ? 512 : 128);
    add_norm_mix_kernel<<<M, threads, smem, stream>>>(a);
    return llmp_check_launch("add_norm_mix");
}

// ------------------------------------------------------------------------------------------
// PolyNorm: out = a N(z) + b N(z^2) + c N(z^3) + e, with N(v) = v / sqrt(mean(v^2) + eps) over a token's F values and the
// powers taken element by element. z float32 or bfloat16; the three mean squares are float32.
// ------------------------------------------------------------------------------------------
__global__ void poly_norm_kernel(const void* __restrict__ z, int z_bf16, long ldz, const float* __restrict__ act, float eps,
                                 void* __restrict__ out, int out_bf16, int F) {
    __shared__ float scratch[32];
    const int n = blockIdx.x;
    const size_t base = (size_t)n * ldz;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int c = threadIdx.x; c < F; c += blockDim.x) {
        const float v = load_dt(z, z_bf16, base + c);
        const float v2 = v * v, v3 = v2 * v;
        s1 += v2;
        s2 += v2 * v2;
        s3 += v3 * v3;
    }
    s1 = block_sum(s1, scratch);
    s2 = block_sum(s2, scratch);
    s3 = block_sum(s3, scratch);
    const float inv = 1.f / (float)F;
    const float r1 = act[0] * rsqrtf(s1 * inv + eps), r2 = act[1] * rsqrtf(s2 * inv + eps), r3 = act[2] * rsqrtf(s3 * inv + eps);
    const float e = act[3];
    for (int c = threadIdx.x; c < F; c += blockDim.x) {
        const float v = load_dt(z, z_bf16, base + c);
        const float v2 = v * v;
        store_dt(out, out_bf16, (size_t)n * F + c, r1 * v + r2 * v2 + r3 * (v2 * v) + e);
    }
}

LLMP_API int llmp_poly_norm(const void* z, int z_dtype, long ldz, const float* act, float eps, void* out, int out_dtype, int N,
                            int F, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(F > 0, "poly_norm: bad width %d", F);
    poly_norm_kernel<<<N, F >= 2048 ? 512 : 128, 0, stream>>>(z, z_dtype == LLMP_BF16, ldz, act, eps, out, out_dtype == LLMP_BF16, F);
    return llmp_check_launch("poly_norm");
}

// ------------------------------------------------------------------------------------------
// Soft cap of the logits, in place: x = cap * tanh(x / cap).
// ------------------------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] * inv_cap);
}

LLMP_API int llmp_softcap(float* x, long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    LLMP_REQUIRE(cap > 0.f, "softcap: the cap must be positive, got %f", (double)cap);
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, (size_t)n, cap, 1.f / cap);
    return llmp_check_launch("softcap");
}
