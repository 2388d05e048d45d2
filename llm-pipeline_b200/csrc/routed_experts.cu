// A feed-forward of many small experts of which every token uses a few.
//   route_topk:      router logits in float32 (float32 copy of the router matrix, the token's row as stored); scores by
//                    sigmoid (each logit alone) or softmax (over all router outputs); the `top` largest of
//                    score (+ a correction per router output, if given); a chosen expert's weight is its score
//                    without the correction. A further row of the matrix, if asked for, gives a gate per token:
//                    sigmoid of its logit.
//   expert_gate_up:  per (token, choice), with w the choice's weight, by the form of the expert:
//                    clamped:  g = min(w (Wg h), limit), u = clamp(w (Wu h), -limit, limit), y = g sigmoid(1.702 g) (u + 1)
//                              (the weight scales the expert's input; the first products are linear, so it is applied to
//                              their float32 sums);
//                    silu:     y = w silu(Wg h) (Wu h) (the weight scales the expert's output; the last product is
//                              linear, so it is applied to the float32 activation before it is rounded).
//   expert_down:     out[token] = sum over the token's choices, in their order, of Wd y (float32). A choice whose id is
//                    not below the number of experts with matrices is an identity expert: it adds w h.
// These kernels read an expert's rows once per token that chose it (a warp per output row): the form for the few
// rows of a decode step. Steps with many rows sort their (token, choice) pairs by expert and take the grouped
// product further down, which reads an expert's rows once per 64 pairs.
#include "common.cuh"

__global__ void route_topk_kernel(const void* __restrict__ h, int h_bf16, const float* __restrict__ wr, int top, int* __restrict__ ids,
                                  float* __restrict__ wts, int Hd, int E, int softmax, const float* __restrict__ correction,
                                  float* __restrict__ gate) {
    extern __shared__ float route_smem[];
    float* logits = route_smem;                              // [E + 1]: logits, then what the choice goes by
    float* score = route_smem + E + 1;                       // [E]: softmax scores (softmax only)
    float* row = route_smem + 2 * E + 1;                     // [Hd]: the token's row, read once
    const int rows_w = gate ? E + 1 : E;                     // the gate's row follows the experts' rows
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < Hd; i += blockDim.x) row[i] = load_as_float(h, h_bf16, (size_t)n * Hd + i);
    __syncthreads();
    for (int e = warp; e < rows_w; e += nwarps) {
        const float* w = wr + (size_t)e * Hd;
        // eight sums a lane, so that eight loads are in flight; their order of addition is fixed
        float acc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] = 0.f;
        int i = lane;
        for (; i + 7 * 32 < Hd; i += 256) {
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[u] = fmaf(row[i + 32 * u], w[i + 32 * u], acc[u]);
        }
        for (; i < Hd; i += 32) acc[0] = fmaf(row[i], w[i], acc[0]);
        const float s = warp_sum(((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7])));
        if (lane == 0) logits[e] = s;
    }
    __syncthreads();
    if (warp == 0) {
        if (gate && lane == 0) gate[n] = 1.f / (1.f + expf(-logits[E]));
        if (softmax) {
            float mx = -INFINITY;
            for (int e = lane; e < E; e += 32) mx = fmaxf(mx, logits[e]);
            mx = warp_max(mx);
            float sum = 0.f;
            for (int e = lane; e < E; e += 32) {
                const float p = expf(logits[e] - mx);
                score[e] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            __syncwarp();
            for (int e = lane; e < E; e += 32) {
                const float p = score[e] / sum;
                score[e] = p;
                logits[e] = correction ? p + correction[e] : p;
            }
            __syncwarp();
        } else if (correction) {
            for (int e = lane; e < E; e += 32) {
                score[e] = 1.f / (1.f + expf(-logits[e]));
                logits[e] = score[e] + correction[e];
            }
            __syncwarp();
        }
        const bool by_score = softmax || correction;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = -1;
            for (int e = lane; e < E; e += 32)
                if (logits[e] > best) { best = logits[e]; at = e; }
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa >= 0 && (at < 0 || oa < at))) { best = ob; at = oa; }
            }
            if (lane == 0) {
                ids[(size_t)n * top + k] = at;
                wts[(size_t)n * top + k] = by_score ? score[at] : 1.f / (1.f + expf(-best));
                logits[at] = -INFINITY;
            }
            __syncwarp();
        }
    }
}

// softmax: 0 sigmoid scores, 1 softmax over the E router outputs. correction: float32 [E] or null. gate: float32 [N] or
// null; when given, w_router has E + 1 rows and gate[n] = sigmoid(row E . h[n]).
LLMP_API int llmp_route_topk(const void* h, int h_dtype, const float* w_router, int top, int* ids, float* wts, int N, int Hd, int E,
                             int softmax, const float* correction, float* gate, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(E > 0 && top > 0 && top <= E && Hd > 0 && E <= 8192, "route_topk: bad sizes experts=%d top=%d width=%d", E, top, Hd);
    const size_t smem = (size_t)(2 * E + 1 + Hd) * sizeof(float);
    LLMP_REQUIRE(smem <= 200 * 1024, "route_topk: a row of %d entries does not fit shared memory", Hd);
    LLMP_ALLOW_SMEM(route_topk_kernel, smem);
    // few rows (a decode step): a warp per expert, so that the router matrix is read by many warps at once
    route_topk_kernel<<<N, N <= 64 ? 1024 : 256, smem, stream>>>(h, h_dtype == LLMP_BF16, w_router, top, ids, wts, Hd, E, softmax,
                                                                  correction, gate);
    return llmp_check_launch("route_topk");
}

// form 0: clamped, the weight on the input; form 1: silu(g) u, the weight on the output
__device__ __forceinline__ float expert_act(float g, float u, float w, float limit, int form) {
    if (form == 1) return w * (g / (1.f + expf(-g))) * u;
    g = fminf(w * g, limit);
    u = fminf(fmaxf(w * u, -limit), limit);
    return g * (1.f / (1.f + expf(-1.702f * g))) * (u + 1.f);
}

// Eight consecutive entries of a row as floats, by 16-byte loads (the rows are 16-byte aligned when their length is a
// multiple of 8 and the tensors are).
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __low2float(h2[i]);
        v[2 * i + 1] = __high2float(h2[i]);
    }
}
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// grid (pairs, ceil(F / 8)): a warp per row of the expert's gate and up matrices (w_gu[e] = [gate rows; up rows]).
// VEC: the rows' length is a multiple of 8; a lane then takes 8 consecutive entries a step, in 16-byte loads.
template <typename T, bool VEC>
__global__ void expert_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gu, const int* __restrict__ ids,
                                      const float* __restrict__ wts, float limit, T* __restrict__ y, int top, int Hd, int F,
                                      int form, int E) {
    const int pair = blockIdx.x;
    const int f = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (f >= F) return;
    const int e = ids[pair];
    if (e >= E) return;                                      // an identity expert has no matrices
    const T* x = h + (size_t)(pair / top) * Hd;
    const T* wg = w_gu + ((size_t)e * 2 * F + f) * Hd;
    const T* wu = wg + (size_t)F * Hd;
    float g = 0.f, u = 0.f;
    if (VEC) {
#pragma unroll 2
        for (int i = lane * 8; i < Hd; i += 256) {
            float xv[8], a[8], b[8];
            load8(x + i, xv);
            load8(wg + i, a);
            load8(wu + i, b);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                g = fmaf(xv[j], a[j], g);
                u = fmaf(xv[j], b[j], u);
            }
        }
    } else {
        for (int i = lane; i < Hd; i += 32) {
            const float xv = to_float(x[i]);
            g = fmaf(xv, to_float(wg[i]), g);
            u = fmaf(xv, to_float(wu[i]), u);
        }
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) y[(size_t)pair * F + f] = from_float<T>(expert_act(g, u, wts[pair], limit, form));
}

// grid (tokens, ceil(Hd / 8)): a warp per output entry, the token's choices added in their order.
template <typename T, bool VEC>
__global__ void expert_down_kernel(const T* __restrict__ y, const T* __restrict__ w_down, const int* __restrict__ ids,
                                   float* __restrict__ out, int top, int Hd, int F, const T* __restrict__ h,
                                   const float* __restrict__ wts, int E) {
    const int n = blockIdx.x;
    const int c = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (c >= Hd) return;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const int pair = n * top + k;
        if (ids[pair] >= E) {                                // identity expert: the weighted input itself
            total += wts[pair] * to_float(h[(size_t)n * Hd + c]);
            continue;
        }
        const T* w = w_down + ((size_t)ids[pair] * Hd + c) * F;
        const T* yv = y + (size_t)pair * F;
        float s = 0.f;
        if (VEC) {
#pragma unroll 2
            for (int i = lane * 8; i < F; i += 256) {
                float a[8], b[8];
                load8(yv + i, a);
                load8(w + i, b);
#pragma unroll
                for (int j = 0; j < 8; ++j) s = fmaf(a[j], b[j], s);
            }
        } else {
            for (int i = lane; i < F; i += 32) s = fmaf(to_float(yv[i]), to_float(w[i]), s);
        }
        total += warp_sum(s);
    }
    if (lane == 0) out[(size_t)n * Hd + c] = total;
}

// form: the expert's form (expert_act). E: experts with matrices; ids from E on are identity experts.
LLMP_API int llmp_expert_rows(const void* h, const void* w_gu, const void* w_down, int dtype, const int* ids, const float* wts,
                              float limit, void* y, float* out, int N, int top, int Hd, int F, int form, int E, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(top > 0 && Hd > 0 && F > 0, "expert_rows: bad sizes top=%d width=%d ff=%d", top, Hd, F);
    LLMP_REQUIRE((F + 7) / 8 <= 65535 && (Hd + 7) / 8 <= 65535, "expert_rows: too wide");
    dim3 g1(N * top, (F + 7) / 8), g2(N, (Hd + 7) / 8);
    const bool aligned = ((size_t)h | (size_t)w_gu | (size_t)w_down | (size_t)y) % 16 == 0;
    const bool v1 = aligned && Hd % 8 == 0, v2 = aligned && F % 8 == 0;
#define LLMP_EXPERT_ROWS(T)                                                                                                        \
    do {                                                                                                                           \
        if (v1) expert_gate_up_kernel<T, true><<<g1, 256, 0, stream>>>((const T*)h, (const T*)w_gu, ids, wts, limit, (T*)y, top, Hd, F, form, E);  \
        else expert_gate_up_kernel<T, false><<<g1, 256, 0, stream>>>((const T*)h, (const T*)w_gu, ids, wts, limit, (T*)y, top, Hd, F, form, E);    \
        if (v2) expert_down_kernel<T, true><<<g2, 256, 0, stream>>>((const T*)y, (const T*)w_down, ids, out, top, Hd, F, (const T*)h, wts, E);                 \
        else expert_down_kernel<T, false><<<g2, 256, 0, stream>>>((const T*)y, (const T*)w_down, ids, out, top, Hd, F, (const T*)h, wts, E);                   \
    } while (0)
    if (dtype == LLMP_F32) LLMP_EXPERT_ROWS(float);
    else LLMP_EXPERT_ROWS(bf16);
#undef LLMP_EXPERT_ROWS
    return llmp_check_launch("expert_rows");
}

// ------------------------------------------------------------------------------------------
// The grouped form for steps of many rows (bfloat16, tensor cores: mma.sync m16n8k16, float32 sums).
//   count / plan / scatter: the (token, choice) pairs are sorted by expert on the device. Every expert's run of pairs
//       starts at a multiple of 64 rows of the sorted order, so a tile of 64 rows has one expert; the places between an
//       expert's last pair and the next multiple of 64 hold -1. Which place within its expert's run a pair gets
//       depends on the order of atomic adds, but a row's result does not depend on its place.
//   grouped products: a block takes a tile of 64 sorted rows and 64 output columns, its four warps 16 rows each.
//       First product: rows gathered from h by pair, against the expert's gate rows and up rows of the same columns,
//       with the activation in the epilogue (y, bfloat16, in sorted order). Second product: y against the expert's
//       down rows, written as float32 at the pair's own place.
//   combine: out[token] = sum of its pairs' rows in the order of its choices.
// ------------------------------------------------------------------------------------------
#define GX_ROWS 64
#define GX_COLS 64
#define GX_K 64
#define GX_STRIDE (GX_K + 8)

// pairs of identity experts (ids from E on) take no part in the sorted order
__global__ void moe_count_kernel(const int* __restrict__ ids, int pairs, int* __restrict__ counts, int E) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < pairs && ids[i] < E) atomicAdd(&counts[ids[i]], 1);
}

// One block. counts[E] -> cursor[E] (first sorted row of each expert), the tile list and its length.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ cursor, int* __restrict__ tile_expert,
                                int* __restrict__ tile_row0, int* __restrict__ num_tiles) {
    if (threadIdx.x != 0) return;
    int row = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
        cursor[e] = row;
        const int n = (counts[e] + GX_ROWS - 1) / GX_ROWS;
        for (int k = 0; k < n; ++k) {
            tile_expert[tiles] = e;
            tile_row0[tiles] = row + k * GX_ROWS;
            ++tiles;
        }
        row += n * GX_ROWS;
    }
    *num_tiles = tiles;
}

__global__ void moe_scatter_kernel(const int* __restrict__ ids, int pairs, int* __restrict__ cursor, int* __restrict__ sorted_pair, int E) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < pairs && ids[i] < E) sorted_pair[atomicAdd(&cursor[ids[i]], 1)] = i;
}

__device__ __forceinline__ void gx_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void gx_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void gx_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct GroupedArgs {
    const bf16* a;            // first product: h [tokens, K]; second: y [sorted rows, K]
    const bf16* w;            // first: [E, 2 cols_total, K]; second: [E, cols_total, K]
    const int* sorted_pair; const int* tile_expert; const int* tile_row0; const int* num_tiles;
    const float* wts;
    bf16* y;                  // first product's result [sorted rows, cols_total]
    float* out;               // second product's result [pairs, cols_total]
    int top, K, cols_total, form;
    float limit;
};

// GATED: the first product (two weight tiles, activation); else the second.
template <bool GATED>
__global__ void __launch_bounds__(128) moe_grouped_kernel(const GroupedArgs a) {
    // two stages of [A tile | weight tile(s)], each tile [64][GX_STRIDE]: the copies of the next K step run under the
    // products of this one
    extern __shared__ __align__(16) unsigned char gx_smem[];
    constexpr int TILES = GATED ? 3 : 2;
    constexpr int STAGE = TILES * GX_ROWS * GX_STRIDE;
    bf16* ring = reinterpret_cast<bf16*>(gx_smem);
    __shared__ int row_pair[GX_ROWS];
    const int tile = blockIdx.x;
    if (tile >= *a.num_tiles) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int e = a.tile_expert[tile], row0 = a.tile_row0[tile];
    const int col0 = blockIdx.y * GX_COLS;
    if (tid < GX_ROWS) row_pair[tid] = a.sorted_pair[row0 + tid];
    __syncthreads();
    const bf16* wg = a.w + ((size_t)e * (GATED ? 2 : 1) * a.cols_total + col0) * a.K;
    const bf16* wu = wg + (size_t)a.cols_total * a.K;
    float cg[8][4], cu[GATED ? 8 : 1][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) cg[i][0] = cg[i][1] = cg[i][2] = cg[i][3] = 0.f;
#pragma unroll
    for (int i = 0; i < (GATED ? 8 : 1); ++i) cu[i][0] = cu[i][1] = cu[i][2] = cu[i][3] = 0.f;

    auto copy_step = [&](int k0, int stage) {
        bf16* As = ring + (size_t)stage * STAGE;
        bf16* Bs = As + GX_ROWS * GX_STRIDE;
        for (int v = tid; v < GX_ROWS * (GX_K / 8); v += 128) {
            const int row = v / (GX_K / 8), c = (v % (GX_K / 8)) * 8;
            const int pair = row_pair[row];
            const bool ok = pair >= 0 && k0 + c < a.K;
            const size_t src_row = GATED ? (size_t)(pair / a.top) : (size_t)(row0 + row);
            gx_cp_async_16(As + row * GX_STRIDE + c, ok ? a.a + src_row * a.K + k0 + c : a.a, ok);
            const bool okw = col0 + row < a.cols_total && k0 + c < a.K;
            gx_cp_async_16(Bs + row * GX_STRIDE + c, okw ? wg + (size_t)row * a.K + k0 + c : a.w, okw);
            if (GATED) gx_cp_async_16(Bs + (GX_COLS + row) * GX_STRIDE + c, okw ? wu + (size_t)row * a.K + k0 + c : a.w, okw);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    copy_step(0, 0);
    int stage = 0;
    for (int k0 = 0; k0 < a.K; k0 += GX_K, stage ^= 1) {
        if (k0 + GX_K < a.K) {
            copy_step(k0 + GX_K, stage ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const bf16* As = ring + (size_t)stage * STAGE;
        const bf16* Bs = As + GX_ROWS * GX_STRIDE;
#pragma unroll
        for (int ks = 0; ks < GX_K / 16; ++ks) {
            unsigned fa[4];
            gx_ldmatrix_x4(fa, As + (warp * 16 + (lane & 15)) * GX_STRIDE + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < 8; nb += 2) {
                unsigned fb[4];
                gx_ldmatrix_x4(fb, Bs + ((nb + (lane >> 4)) * 8 + (lane & 7)) * GX_STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
                gx_mma(cg[nb], fa, fb[0], fb[1]);
                gx_mma(cg[nb + 1], fa, fb[2], fb[3]);
                if (GATED) {
                    gx_ldmatrix_x4(fb, Bs + (GX_COLS + (nb + (lane >> 4)) * 8 + (lane & 7)) * GX_STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
                    gx_mma(cu[nb], fa, fb[0], fb[1]);
                    gx_mma(cu[nb + 1], fa, fb[2], fb[3]);
                }
            }
        }
        __syncthreads();                                         // the stage may be overwritten by the copies after next
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int row = warp * 16 + g + 8 * h2;
        const int pair = row_pair[row];
        if (pair < 0) continue;
        const float w = GATED ? a.wts[pair] : 0.f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int c2 = 0; c2 < 2; ++c2) {
                const int col = col0 + nb * 8 + 2 * t + c2;
                if (col >= a.cols_total) continue;
                if (GATED) a.y[(size_t)(row0 + row) * a.cols_total + col] = __float2bfloat16_rn(expert_act(cg[nb][2 * h2 + c2], cu[GATED ? nb : 0][2 * h2 + c2], w, a.limit, a.form));
                else a.out[(size_t)pair * a.cols_total + col] = cg[nb][2 * h2 + c2];
            }
        }
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ pair_out, float* __restrict__ out, int top, int Hd, size_t total,
                                   const int* __restrict__ ids, const float* __restrict__ wts, const bf16* __restrict__ h, int E) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t n = i / Hd, c = i % Hd;
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
        const size_t pair = n * top + k;
        s += ids[pair] < E ? pair_out[pair * Hd + c] : wts[pair] * __bfloat162float(h[i]);     // identity expert: w h
    }
    out[i] = s;
}

LLMP_API int llmp_expert_grouped_supports(int Hd, int F) { return Hd % 8 == 0 && F % 8 == 0; }

// Rows of the sorted order for `pairs` pairs among E experts (every expert's run padded to a multiple of 64).
LLMP_API long llmp_expert_grouped_rows(int pairs, int E) { return ((long)(pairs + GX_ROWS - 1) / GX_ROWS + E) * GX_ROWS; }

// ints: int32 scratch [3 E + 1 + 2 tiles_max + rows_max] with tiles_max = rows_max / 64; y: bf16 [rows_max, F];
// pair_out: float32 [pairs, Hd] (unused when top == 1 and there are no identity experts: the rows go straight to out).
// form: the expert's form (expert_act). identity: ids E .. E + identity - 1 are identity experts.
LLMP_API int llmp_expert_grouped(const void* h, const void* w_gu, const void* w_down, const int* ids, const float* wts, float limit,
                                 int* ints, void* y, float* pair_out, float* out, int N, int top, int Hd, int F, int E, int form,
                                 int identity, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(llmp_expert_grouped_supports(Hd, F) && top > 0 && E > 0, "expert_grouped: sizes width=%d ff=%d are not served", Hd, F);
    const int pairs = N * top;
    const long rows_max = llmp_expert_grouped_rows(pairs, E);
    const int tiles_max = (int)(rows_max / GX_ROWS);
    int* counts = ints;
    int* cursor = ints + E;
    int* num_tiles = ints + 2 * E;
    int* tile_expert = ints + 2 * E + 1;
    int* tile_row0 = tile_expert + tiles_max;
    int* sorted_pair = tile_row0 + tiles_max;
    cudaMemsetAsync(counts, 0, sizeof(int) * E, stream);
    cudaMemsetAsync(sorted_pair, 0xFF, sizeof(int) * rows_max, stream);
    moe_count_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(ids, pairs, counts, E);
    moe_plan_kernel<<<1, 32, 0, stream>>>(counts, E, cursor, tile_expert, tile_row0, num_tiles);
    moe_scatter_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(ids, pairs, cursor, sorted_pair, E);
    GroupedArgs a;
    a.sorted_pair = sorted_pair; a.tile_expert = tile_expert; a.tile_row0 = tile_row0; a.num_tiles = num_tiles;
    a.wts = wts; a.y = (bf16*)y; a.top = top; a.limit = limit; a.form = form;
    const bool combine = top > 1 || identity > 0;
    LLMP_REQUIRE(!combine || pair_out, "expert_grouped: the sum over a token's choices needs its scratch");
    a.a = (const bf16*)h; a.w = (const bf16*)w_gu; a.K = Hd; a.cols_total = F; a.out = nullptr;
    const size_t smem_gated = sizeof(bf16) * 2 * 3 * GX_ROWS * GX_STRIDE, smem_plain = sizeof(bf16) * 2 * 2 * GX_ROWS * GX_STRIDE;
    LLMP_ALLOW_SMEM(moe_grouped_kernel<true>, smem_gated);
    moe_grouped_kernel<true><<<dim3(tiles_max, (F + GX_COLS - 1) / GX_COLS), 128, smem_gated, stream>>>(a);
    a.a = (const bf16*)y; a.w = (const bf16*)w_down; a.K = F; a.cols_total = Hd; a.out = combine ? pair_out : out;
    LLMP_ALLOW_SMEM(moe_grouped_kernel<false>, smem_plain);
    moe_grouped_kernel<false><<<dim3(tiles_max, (Hd + GX_COLS - 1) / GX_COLS), 128, smem_plain, stream>>>(a);
    if (combine) {
        const size_t total = (size_t)N * Hd;
        moe_combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(pair_out, out, top, Hd, total, ids, wts, (const bf16*)h, E);
    }
    return llmp_check_launch("expert_grouped");
}
