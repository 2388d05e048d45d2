// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores with float32 accumulation.
// This is the matrix product of the true 32-bit path (no tensor core, no reduced-precision
// mode) and accepts every size. Each output element adds its K products in ascending k, so a
// row's result does not depend on how many other rows are in the call.
#include "common.cuh"

#define GT_BM 64
#define GT_BN 64
#define GT_BK 16

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const TI* __restrict__ A, const TI* __restrict__ W, const void* __restrict__ bias, int bias_bf16,
               TO* __restrict__ C, int M, int N, int K, long lda, long ldw, long ldc, long batch_a = 0, long batch_w = 0,
               long batch_c = 0) {
    // blockIdx.z counts the products of a batch: each has its own A, W and C, the given strides apart
    A += (size_t)blockIdx.z * batch_a;
    W += (size_t)blockIdx.z * batch_w;
    C += (size_t)blockIdx.z * batch_c;
    __shared__ float As[GT_BK][GT_BM + 4];
    __shared__ float Ws[GT_BK][GT_BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GT_BM, n0 = blockIdx.x * GT_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GT_BK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = tid + 256 * r;
            const int row = e >> 4, col = e & 15;
            const int k = k0 + col;
            const int m = m0 + row, n = n0 + row;
            As[col][row] = (m < M && k < K) ? to_float(A[(size_t)m * lda + k]) : 0.f;
            Ws[col][row] = (n < N && k < K) ? to_float(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GT_BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_as_float(bias, bias_bf16, n);
            C[(size_t)m * ldc + n] = from_float<TO>(v);
        }
    }
}

// in_dtype: type of A and W.  out_dtype: type of C (float32, or the input type).
LLMP_API int llmp_gemm_simt(const void* A, const void* W, const void* bias, int bias_dtype, void* C, int in_dtype,
                            int out_dtype, int M, int N, int K, long lda, long ldw, long ldc, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    LLMP_REQUIRE(K > 0, "gemm: bad K %d", K);
    LLMP_REQUIRE((M + GT_BM - 1) / GT_BM <= 65535, "gemm: too many rows %d", M);
    dim3 grid((N + GT_BN - 1) / GT_BN, (M + GT_BM - 1) / GT_BM);
    const int bb = bias_dtype == LLMP_BF16;
    if (in_dtype == LLMP_F32 && out_dtype == LLMP_F32)
        gemm_nt_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)A, (const float*)W, bias, bb, (float*)C,
                                                               M, N, K, lda, ldw, ldc);
    else if (in_dtype == LLMP_BF16 && out_dtype == LLMP_BF16)
        gemm_nt_kernel<bf16, bf16><<<grid, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, bias, bb, (bf16*)C, M, N,
                                                             K, lda, ldw, ldc);
    else if (in_dtype == LLMP_BF16 && out_dtype == LLMP_F32)
        gemm_nt_kernel<bf16, float><<<grid, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, bias, bb, (float*)C, M,
                                                              N, K, lda, ldw, ldc);
    else {
        llmp_set_error("gemm: unsupported type combination in=%d out=%d", in_dtype, out_dtype);
        return 1;
    }
    return llmp_check_launch("gemm_simt");
}

// The same batch for at most 16 rows a product (a decode step): a warp per output column reads the column's weight
// row once and keeps one sum per row of A; the K products of a sum are added lane by lane in ascending k, then across
// the lanes in a fixed order.
#define GR_MAX_ROWS 16
__device__ __forceinline__ void gr_load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __low2float(h2[i]);
        v[2 * i + 1] = __high2float(h2[i]);
    }
}
__device__ __forceinline__ void gr_load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// VEC: K, the strides and the addresses allow 16-byte loads of 8 consecutive entries.
template <typename TI, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
gemm_rows_kernel(const TI* __restrict__ A, const TI* __restrict__ W, TO* __restrict__ C, int M, int N, int K, long lda, long ldw,
                 long ldc, long batch_a, long batch_w, long batch_c) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    A += (size_t)blockIdx.y * batch_a;
    C += (size_t)blockIdx.y * batch_c;
    const TI* w = W + (size_t)blockIdx.y * batch_w + (size_t)n * ldw;
    float acc[GR_MAX_ROWS];
#pragma unroll
    for (int m = 0; m < GR_MAX_ROWS; ++m) acc[m] = 0.f;
    if (VEC) {
        for (int k = lane * 8; k < K; k += 256) {
            float wv[8];
            gr_load8(w + k, wv);
#pragma unroll
            for (int m = 0; m < GR_MAX_ROWS; ++m) {
                if (m < M) {
                    float xv[8];
                    gr_load8(A + (size_t)m * lda + k, xv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[m] = fmaf(xv[j], wv[j], acc[m]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = to_float(w[k]);
#pragma unroll
            for (int m = 0; m < GR_MAX_ROWS; ++m)
                if (m < M) acc[m] = fmaf(to_float(A[(size_t)m * lda + k]), wv, acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < GR_MAX_ROWS; ++m) {
        if (m < M) {
            const float v = warp_sum(acc[m]);
            if (lane == 0) C[(size_t)m * ldc + n] = from_float<TO>(v);
        }
    }
}

// A batch of such products in one launch: product b reads A + b * batch_a and W + b * batch_w and writes C + b * batch_c
// (strides in elements; rows of any of them may lie further apart than they are long, so one product per head
// can read and write the heads of a [tokens, heads, size] tensor in place).
LLMP_API int llmp_gemm_simt_batched(const void* A, const void* W, void* C, int in_dtype, int out_dtype, int batch, int M, int N,
                                    int K, long lda, long ldw, long ldc, long batch_a, long batch_w, long batch_c,
                                    cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    LLMP_REQUIRE(K > 0, "batched gemm: bad K %d", K);
    LLMP_REQUIRE((M + GT_BM - 1) / GT_BM <= 65535 && batch <= 65535, "batched gemm: too many rows %d or products %d", M, batch);
    if (M <= GR_MAX_ROWS && (N + 7) / 8 <= 65535) {
        dim3 rows_grid((N + 7) / 8, batch);
        const size_t esize = in_dtype == LLMP_F32 ? 4 : 2;
        const bool vec = K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && batch_a % 8 == 0 && batch_w % 8 == 0 &&
                         ((size_t)A | (size_t)W) % 16 == 0 && esize > 0;
#define LLMP_ROWS(TI, TO)                                                                                                         \
    do {                                                                                                                          \
        if (vec) gemm_rows_kernel<TI, TO, true><<<rows_grid, 256, 0, stream>>>((const TI*)A, (const TI*)W, (TO*)C, M, N, K, lda, ldw,   \
                                                                               ldc, batch_a, batch_w, batch_c);                  \
        else gemm_rows_kernel<TI, TO, false><<<rows_grid, 256, 0, stream>>>((const TI*)A, (const TI*)W, (TO*)C, M, N, K, lda, ldw, ldc, \
                                                                            batch_a, batch_w, batch_c);                          \
    } while (0)
        if (in_dtype == LLMP_F32 && out_dtype == LLMP_F32) LLMP_ROWS(float, float);
        else if (in_dtype == LLMP_BF16 && out_dtype == LLMP_BF16) LLMP_ROWS(bf16, bf16);
        else if (in_dtype == LLMP_BF16 && out_dtype == LLMP_F32) LLMP_ROWS(bf16, float);
        else {
            llmp_set_error("batched gemm: unsupported type combination in=%d out=%d", in_dtype, out_dtype);
            return 1;
        }
#undef LLMP_ROWS
        return llmp_check_launch("gemm_simt_batched (rows)");
    }
    dim3 grid((N + GT_BN - 1) / GT_BN, (M + GT_BM - 1) / GT_BM, batch);
    if (in_dtype == LLMP_F32 && out_dtype == LLMP_F32)
        gemm_nt_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)A, (const float*)W, nullptr, 0, (float*)C, M, N, K,
                                                               lda, ldw, ldc, batch_a, batch_w, batch_c);
    else if (in_dtype == LLMP_BF16 && out_dtype == LLMP_BF16)
        gemm_nt_kernel<bf16, bf16><<<grid, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, nullptr, 0, (bf16*)C, M, N, K, lda,
                                                             ldw, ldc, batch_a, batch_w, batch_c);
    else if (in_dtype == LLMP_BF16 && out_dtype == LLMP_F32)
        gemm_nt_kernel<bf16, float><<<grid, 256, 0, stream>>>((const bf16*)A, (const bf16*)W, nullptr, 0, (float*)C, M, N, K,
                                                              lda, ldw, ldc, batch_a, batch_w, batch_c);
    else {
        llmp_set_error("batched gemm: unsupported type combination in=%d out=%d", in_dtype, out_dtype);
        return 1;
    }
    return llmp_check_launch("gemm_simt_batched");
}
