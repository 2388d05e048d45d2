// Kernels of blocks whose sublayers run side by side on one normed input, and of their feed-forwards:
//   add_layernorm:   residual (float32, in place) += addend a + addend b (each float32 or bfloat16, either may be
//                    absent), then out = (x - mean) / sqrt(var + eps) * w + b with var the mean of the squared
//                    deviations, all float32, rounded once to the output type. With `rows` only those rows are
//                    computed and the residual stays as it is (the head's rows).
//   relu_squared:    out = max(z, 0)^2.
//   add_scaled_rows: out[n, :] += s[n] * x[n, :] (float32 out and s).
// A row's sums are added in an order that the row length fixes, so a row's result does not depend on the step.
#include "common.cuh"

#define LN_THREADS 256

__device__ __forceinline__ void ln_load4(const void* p, int is_bf16, size_t i, float (&v)[4]) {
    if (is_bf16) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        v[0] = __low2float(h2[0]); v[1] = __high2float(h2[0]); v[2] = __low2float(h2[1]); v[3] = __high2float(h2[1]);
    } else {
        const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
}

__device__ __forceinline__ void ln_store4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void ln_store4(bf16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// PIECES: 4-entry pieces a thread keeps in registers (H <= 4 * LN_THREADS * PIECES); VEC: H is a multiple of 4 and every
// pointer is 16-byte aligned. Without VEC the row goes through shared memory entry by entry.
template <typename TO, int PIECES>
__global__ void __launch_bounds__(LN_THREADS)
add_layernorm_vec_kernel(float* __restrict__ residual, const void* __restrict__ da, int da_bf16, const void* __restrict__ db, int db_bf16,
                         const void* __restrict__ w, const void* __restrict__ b, int wb_bf16, float eps, TO* __restrict__ out, int H,
                         const int* __restrict__ rows) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x;
    const size_t row = rows ? (size_t)rows[r] : (size_t)r;
    float x[PIECES][4];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < PIECES; ++k) {
        const int c = (threadIdx.x + k * LN_THREADS) * 4;
        x[k][0] = x[k][1] = x[k][2] = x[k][3] = 0.f;
        if (c < H) {
            ln_load4(residual, 0, row * H + c, x[k]);
            float t[4];
            if (da) {
                ln_load4(da, da_bf16, row * H + c, t);
#pragma unroll
                for (int i = 0; i < 4; ++i) x[k][i] += t[i];
            }
            if (db) {
                ln_load4(db, db_bf16, row * H + c, t);
#pragma unroll
                for (int i = 0; i < 4; ++i) x[k][i] += t[i];
            }
            if (!rows && (da || db)) ln_store4(residual + row * H + c, x[k]);
            sum += (x[k][0] + x[k][1]) + (x[k][2] + x[k][3]);
        }
    }
    const float mean = block_sum(sum, scratch) / (float)H;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < PIECES; ++k) {
        const int c = (threadIdx.x + k * LN_THREADS) * 4;
        if (c < H) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                x[k][i] -= mean;
                sq = fmaf(x[k][i], x[k][i], sq);
            }
        }
    }
    const float rstd = rsqrtf(block_sum(sq, scratch) / (float)H + eps);
#pragma unroll
    for (int k = 0; k < PIECES; ++k) {
        const int c = (threadIdx.x + k * LN_THREADS) * 4;
        if (c < H) {
            float wv[4], bv[4], y[4];
            ln_load4(w, wb_bf16, c, wv);
            ln_load4(b, wb_bf16, c, bv);
#pragma unroll
            for (int i = 0; i < 4; ++i) y[i] = fmaf(x[k][i] * rstd, wv[i], bv[i]);
            ln_store4(out + (size_t)r * H + c, y);
        }
    }
}

template <typename TO>
__global__ void __launch_bounds__(LN_THREADS)
add_layernorm_kernel(float* __restrict__ residual, const void* __restrict__ da, int da_bf16, const void* __restrict__ db, int db_bf16,
                     const void* __restrict__ w, const void* __restrict__ b, int wb_bf16, float eps, TO* __restrict__ out, int H,
                     const int* __restrict__ rows) {
    extern __shared__ float ln_row[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t row = rows ? (size_t)rows[r] : (size_t)r;
    float sum = 0.f;
    for (int c = threadIdx.x; c < H; c += LN_THREADS) {
        float v = residual[row * H + c];
        if (da) v += load_as_float(da, da_bf16, row * H + c);
        if (db) v += load_as_float(db, db_bf16, row * H + c);
        if (!rows && (da || db)) residual[row * H + c] = v;
        ln_row[c] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)H;
    float sq = 0.f;
    for (int c = threadIdx.x; c < H; c += LN_THREADS) {
        const float v = ln_row[c] - mean;
        sq = fmaf(v, v, sq);
    }
    const float rstd = rsqrtf(block_sum(sq, scratch) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += LN_THREADS)
        out[(size_t)r * H + c] = from_float<TO>(fmaf((ln_row[c] - mean) * rstd, load_as_float(w, wb_bf16, c), load_as_float(b, wb_bf16, c)));
}

LLMP_API int llmp_add_layernorm(float* residual, const void* da, int da_dtype, const void* db, int db_dtype, const void* w, const void* b,
                                int wb_dtype, float eps, void* out, int out_dtype, int R, int H, const int* rows, cudaStream_t stream) {
    if (R <= 0) return 0;
    LLMP_REQUIRE(H > 0, "add_layernorm: bad width %d", H);
    const int a_bf = da_dtype == LLMP_BF16, b_bf = db_dtype == LLMP_BF16, wb_bf = wb_dtype == LLMP_BF16;
    const bool aligned = (((size_t)residual | (size_t)da | (size_t)db | (size_t)w | (size_t)b | (size_t)out) % 16) == 0;
    const int pieces = (H / 4 + LN_THREADS - 1) / LN_THREADS;
    if (aligned && H % 4 == 0 && pieces <= 8) {
#define LLMP_LN_VEC(TO, P)                                                                                                         \
    cudaError_t e = llmp_launch_dependent(add_layernorm_vec_kernel<TO, P>, dim3(R), dim3(LN_THREADS), 0, stream, residual, da, a_bf, \
                                          db, b_bf, w, b, wb_bf, eps, (TO*)out, H, rows);                                         \
    if (e != cudaSuccess) { llmp_set_error("add_layernorm: %s", cudaGetErrorString(e)); return 1; }
#define LLMP_LN_PIECES(TO)                                           \
    do {                                                             \
        if (pieces <= 1) { LLMP_LN_VEC(TO, 1) }                      \
        else if (pieces <= 2) { LLMP_LN_VEC(TO, 2) }                 \
        else if (pieces <= 4) { LLMP_LN_VEC(TO, 4) }                 \
        else { LLMP_LN_VEC(TO, 8) }                                  \
    } while (0)
        if (out_dtype == LLMP_F32) LLMP_LN_PIECES(float);
        else LLMP_LN_PIECES(bf16);
#undef LLMP_LN_PIECES
#undef LLMP_LN_VEC
        return llmp_check_launch("add_layernorm");
    }
    const size_t smem = (size_t)H * sizeof(float);
    LLMP_REQUIRE(smem <= 200 * 1024, "add_layernorm: a row of %d entries does not fit shared memory", H);
    if (out_dtype == LLMP_F32) {
        LLMP_ALLOW_SMEM(add_layernorm_kernel<float>, smem);
        add_layernorm_kernel<float><<<R, LN_THREADS, smem, stream>>>(residual, da, a_bf, db, b_bf, w, b, wb_bf, eps, (float*)out, H, rows);
    } else {
        LLMP_ALLOW_SMEM(add_layernorm_kernel<bf16>, smem);
        add_layernorm_kernel<bf16><<<R, LN_THREADS, smem, stream>>>(residual, da, a_bf, db, b_bf, w, b, wb_bf, eps, (bf16*)out, H, rows);
    }
    return llmp_check_launch("add_layernorm");
}

template <typename T>
__global__ void relu_squared_kernel(const T* z, T* out, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float v = fmaxf(to_float(z[i]), 0.f);
    out[i] = from_float<T>(v * v);
}

// eight bfloat16 entries a thread, in 16-byte pieces
__global__ void relu_squared_bf16x8_kernel(const uint4* z, uint4* out, size_t pieces) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pieces) return;
    uint4 raw = z[i];
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float a = fmaxf(__low2float(h2[k]), 0.f), b = fmaxf(__high2float(h2[k]), 0.f);
        h2[k] = __floats2bfloat162_rn(a * a, b * b);
    }
    out[i] = raw;
}

LLMP_API int llmp_relu_squared(const void* z, void* out, int dtype, long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (dtype == LLMP_BF16 && total % 8 == 0 && (((size_t)z | (size_t)out) % 16) == 0) {
        const size_t pieces = (size_t)total / 8;
        relu_squared_bf16x8_kernel<<<(unsigned)((pieces + 255) / 256), 256, 0, stream>>>((const uint4*)z, (uint4*)out, pieces);
    } else if (dtype == LLMP_BF16) {
        relu_squared_kernel<bf16><<<(unsigned)(((size_t)total + 255) / 256), 256, 0, stream>>>((const bf16*)z, (bf16*)out, (size_t)total);
    } else {
        relu_squared_kernel<float><<<(unsigned)(((size_t)total + 255) / 256), 256, 0, stream>>>((const float*)z, (float*)out, (size_t)total);
    }
    return llmp_check_launch("relu_squared");
}

template <typename T>
__global__ void add_scaled_rows_kernel(float* __restrict__ out, const T* __restrict__ x, const float* __restrict__ s, int H, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    out[i] = fmaf(s[i / H], to_float(x[i]), out[i]);
}

LLMP_API int llmp_add_scaled_rows(float* out, const void* x, int x_dtype, const float* s, int N, int H, cudaStream_t stream) {
    if (N <= 0 || H <= 0) return 0;
    const size_t total = (size_t)N * H;
    if (x_dtype == LLMP_BF16)
        add_scaled_rows_kernel<bf16><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(out, (const bf16*)x, s, H, total);
    else
        add_scaled_rows_kernel<float><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(out, (const float*)x, s, H, total);
    return llmp_check_launch("add_scaled_rows");
}
