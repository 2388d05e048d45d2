// A feed-forward of many small experts of which every token uses a few.
//   route_topk:      router logits in float32 (float32 copy of the router matrix, the token's row as stored), sigmoid
//                    scores, the `top` largest; a chosen expert's weight is its score.
//   expert_gate_up:  per (token, choice): g = min(w (Wg h), limit), u = clamp(w (Wu h), -limit, limit),
//                    y = g sigmoid(1.702 g) (u + 1). The weight scales the expert's input; as the first products are
//                    linear, it is applied to their float32 sums instead.
//   expert_down:     out[token] = sum over the token's choices, in their order, of Wd y (float32).
// These kernels read an expert's rows once per token that chose it (a warp per output row): the form for the few
// rows of a decode step. Steps with many rows sort their (token, choice) pairs by expert and take the grouped
// product further down, which reads an expert's rows once per 64 pairs.
#include "common.cuh"

__global__ void route_topk_kernel(const void* __restrict__ h, int h_bf16, const float* __restrict__ wr, int top, int* __restrict__ ids,
                                  float* __restrict__ wts, int Hd, int E) {
    extern __shared__ float logits[];                        // [E]
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int e = warp; e < E; e += nwarps) {
        const float* w = wr + (size_t)e * Hd;
        float s = 0.f;
        for (int i = lane; i < Hd; i += 32) s = fmaf(load_as_float(h, h_bf16, (size_t)n * Hd + i), w[i], s);
        s = warp_sum(s);
        if (lane == 0) logits[e] = s;
    }
    __syncthreads();
    if (warp == 0) {
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
                wts[(size_t)n * top + k] = 1.f / (1.f + expf(-best));
                logits[at] = -INFINITY;
            }
            __syncwarp();
        }
    }
}

LLMP_API int llmp_route_topk(const void* h, int h_dtype, const float* w_router, int top, int* ids, float* wts, int N, int Hd, int E,
                             cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(E > 0 && top > 0 && top <= E && Hd > 0 && E <= 8192, "route_topk: bad sizes experts=%d top=%d width=%d", E, top, Hd);
    route_topk_kernel<<<N, 128, (size_t)E * sizeof(float), stream>>>(h, h_dtype == LLMP_BF16, w_router, top, ids, wts, Hd, E);
    return llmp_check_launch("route_topk");
}

__device__ __forceinline__ float expert_act(float g, float u, float w, float limit) {
    g = fminf(w * g, limit);
    u = fminf(fmaxf(w * u, -limit), limit);
    return g * (1.f / (1.f + expf(-1.702f * g))) * (u + 1.f);
}

// grid (pairs, ceil(F / 8)): a warp per row of the expert's gate and up matrices (w_gu[e] = [gate rows; up rows]).
template <typename T>
__global__ void expert_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gu, const int* __restrict__ ids,
                                      const float* __restrict__ wts, float limit, T* __restrict__ y, int top, int Hd, int F) {
    const int pair = blockIdx.x;
    const int f = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (f >= F) return;
    const int e = ids[pair];
    const T* x = h + (size_t)(pair / top) * Hd;
    const T* wg = w_gu + ((size_t)e * 2 * F + f) * Hd;
    const T* wu = wg + (size_t)F * Hd;
    float g = 0.f, u = 0.f;
    for (int i = lane; i < Hd; i += 32) {
        const float xv = to_float(x[i]);
        g = fmaf(xv, to_float(wg[i]), g);
        u = fmaf(xv, to_float(wu[i]), u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) y[(size_t)pair * F + f] = from_float<T>(expert_act(g, u, wts[pair], limit));
}

// grid (tokens, ceil(Hd / 8)): a warp per output entry, the token's choices added in their order.
template <typename T>
__global__ void expert_down_kernel(const T* __restrict__ y, const T* __restrict__ w_down, const int* __restrict__ ids,
                                   float* __restrict__ out, int top, int Hd, int F) {
    const int n = blockIdx.x;
    const int c = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (c >= Hd) return;
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        const int pair = n * top + k;
        const T* w = w_down + ((size_t)ids[pair] * Hd + c) * F;
        const T* yv = y + (size_t)pair * F;
        float s = 0.f;
        for (int i = lane; i < F; i += 32) s = fmaf(to_float(yv[i]), to_float(w[i]), s);
        total += warp_sum(s);
    }
    if (lane == 0) out[(size_t)n * Hd + c] = total;
}

LLMP_API int llmp_expert_rows(const void* h, const void* w_gu, const void* w_down, int dtype, const int* ids, const float* wts,
                              float limit, void* y, float* out, int N, int top, int Hd, int F, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(top > 0 && Hd > 0 && F > 0, "expert_rows: bad sizes top=%d width=%d ff=%d", top, Hd, F);
    LLMP_REQUIRE((F + 7) / 8 <= 65535 && (Hd + 7) / 8 <= 65535, "expert_rows: too wide");
    dim3 g1(N * top, (F + 7) / 8), g2(N, (Hd + 7) / 8);
    if (dtype == LLMP_F32) {
        expert_gate_up_kernel<float><<<g1, 256, 0, stream>>>((const float*)h, (const float*)w_gu, ids, wts, limit, (float*)y, top, Hd, F);
        expert_down_kernel<float><<<g2, 256, 0, stream>>>((const float*)y, (const float*)w_down, ids, out, top, Hd, F);
    } else {
        expert_gate_up_kernel<bf16><<<g1, 256, 0, stream>>>((const bf16*)h, (const bf16*)w_gu, ids, wts, limit, (bf16*)y, top, Hd, F);
        expert_down_kernel<bf16><<<g2, 256, 0, stream>>>((const bf16*)y, (const bf16*)w_down, ids, out, top, Hd, F);
    }
    return llmp_check_launch("expert_rows");
}
