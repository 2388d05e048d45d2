// minGRU: a gated recurrence whose gate and candidate read the current token only.
//   z = sigmoid(pz + bz),  u = px + bx,  candidate = u >= 0 ? u + 1/2 : sigmoid(u)
//   S_t = (1 - z) S_(t-1) + z candidate,      y_t = S_t * silu(pg)
// pz, px, pg are the three thirds of one float32 product [tokens, 3 W]; state, gates and the recurrence are float32.
//
// State of a request: two vectors, state[slot][parity][W]. A step that begins at position p reads the vector of
// parity (p - 1) & 1 and, ending at position q, writes the one of parity q & 1: a step of one token never writes the
// vector it read, so running it again gives the same result (a captured decode step may be replayed).
//
// Since the recurrence is linear in S, S_end = A S_begin + B over any run of tokens, with A = prod(1 - z) and B the
// run's result from S_begin = 0. Long portions are cut into chunks of SCAN_CHUNK tokens (short ones, so that a
// prompt of a few thousand tokens gives every SM its fill of warps): a first kernel leaves (A, B)
// of every chunk, a second one walks the chunks of a request and leaves the state before each, a third one runs the
// tokens of every chunk from there, so the tokens of a portion run in parallel. Short portions (decode steps) take one kernel that walks its tokens in order.
#include "common.cuh"

#define SCAN_CHUNK 32

// 1 / (1 + e^-x) with a correctly rounded reciprocal (one special-function instruction and a fix-up, not a division)
__device__ __forceinline__ float sigmoidf_(float x) { return __frcp_rn(1.f + expf(-x)); }

struct GruArgs {
    const float* p;          // [N, 3 W]
    const float* bias;       // [2 W]: bz then bx
    const int* q_start;      // [R + 1]
    const int* slots;        // [R]
    const int* positions;    // [N]
    float* state;            // [slots, 2, W]
    void* out; int out_bf16; // [N, W]
    float* chunk_a; float* chunk_b;   // [R, chunks, W] (chunked path): A and B of every chunk
    float* chunk_s;                   // [R, chunks, W]: the state before every chunk
    int W, chunks;
};

// One token of one channel. The pointers are local and restricted, so that the loads of the next tokens need not wait
// for this token's store: an unrolled loop keeps several rows of the products in flight.
template <typename TO>
__device__ __forceinline__ void gru_token(const float* __restrict__ p, TO* __restrict__ out, size_t row, int W, int c, float bz,
                                          float bx, float& s) {
    const float* pr = p + row * 3 * W;
    const float z = sigmoidf_(pr[c] + bz);
    const float u = pr[W + c] + bx;
    const float g = pr[2 * W + c];
    const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
    s = (1.f - z) * s + z * cand;
    out[row * W + c] = from_float<TO>(s * (g * sigmoidf_(g)));
}

// One thread per (request, channel): walks the request's tokens of this step in order.
template <typename TO>
__global__ void min_gru_serial_kernel(const GruArgs a) {
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= a.W) return;
    const int t0 = a.q_start[r], t1 = a.q_start[r + 1];
    if (t1 <= t0) return;
    const int p0 = a.positions[t0];
    float* st = a.state + (size_t)a.slots[r] * 2 * a.W;
    float s = st[((p0 + 1) & 1) * a.W + c];
    const float bz = a.bias[c], bx = a.bias[a.W + c];
    const float* __restrict__ p = a.p;
    TO* __restrict__ out = reinterpret_cast<TO*>(a.out);
#pragma unroll 4
    for (int t = t0; t < t1; ++t) gru_token<TO>(p, out, t, a.W, c, bz, bx, s);
    st[((p0 + t1 - t0 - 1) & 1) * a.W + c] = s;
}

// Chunked path, first kernel: (A, B) of chunk k of request r for every channel.
__global__ void min_gru_chunk_kernel(const GruArgs a) {
    const int r = blockIdx.x, k = blockIdx.y;
    const int c = blockIdx.z * blockDim.x + threadIdx.x;
    if (c >= a.W) return;
    const int t0 = a.q_start[r] + k * SCAN_CHUNK, end = a.q_start[r + 1];
    if (t0 >= end) return;
    const int t1 = min(end, t0 + SCAN_CHUNK);
    const float bz = a.bias[c], bx = a.bias[a.W + c];
    float A = 1.f, B = 0.f;
    const float* __restrict__ p = a.p;
#pragma unroll 8
    for (int t = t0; t < t1; ++t) {
        const float z = sigmoidf_(p[(size_t)t * 3 * a.W + c] + bz);
        const float u = p[(size_t)t * 3 * a.W + a.W + c] + bx;
        const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
        A *= 1.f - z;
        B = (1.f - z) * B + z * cand;
    }
    const size_t at = ((size_t)r * a.chunks + k) * a.W + c;
    a.chunk_a[at] = A;
    a.chunk_b[at] = B;
}

// Chunked path, second kernel: one thread per (request, channel) walks the request's chunks in order, leaves the state
// before every chunk, and leaves the request's new state. It is the only kernel of the chunked
// path that touches the state, and it reads before it writes, so an even number of tokens (same vector read and
// written) is no hazard.
__global__ void min_gru_prefix_kernel(const GruArgs a) {
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= a.W) return;
    const int begin = a.q_start[r], end = a.q_start[r + 1];
    const int n = end - begin;
    if (n <= 0) return;
    const int p0 = a.positions[begin];
    float* st = a.state + (size_t)a.slots[r] * 2 * a.W;
    float s = st[((p0 + 1) & 1) * a.W + c];
    const int chunks = (n + SCAN_CHUNK - 1) / SCAN_CHUNK;
    const float* __restrict__ As = a.chunk_a;
    const float* __restrict__ Bs = a.chunk_b;
    float* __restrict__ Ss = a.chunk_s;
#pragma unroll 8
    for (int k = 0; k < chunks; ++k) {
        const size_t at = ((size_t)r * a.chunks + k) * a.W + c;
        Ss[at] = s;
        s = As[at] * s + Bs[at];
    }
    st[((p0 + n - 1) & 1) * a.W + c] = s;
}

// Chunked path, third kernel: the chunk's tokens from the state before the chunk.
template <typename TO>
__global__ void min_gru_apply_kernel(const GruArgs a) {
    const int r = blockIdx.x, k = blockIdx.y;
    const int c = blockIdx.z * blockDim.x + threadIdx.x;
    if (c >= a.W) return;
    const int end = a.q_start[r + 1];
    const int t0 = a.q_start[r] + k * SCAN_CHUNK;
    if (t0 >= end) return;
    const int t1 = min(end, t0 + SCAN_CHUNK);
    float s = a.chunk_s[((size_t)r * a.chunks + k) * a.W + c];
    const float bz = a.bias[c], bx = a.bias[a.W + c];
    const float* __restrict__ p = a.p;
    TO* __restrict__ out = reinterpret_cast<TO*>(a.out);
#pragma unroll 8
    for (int t = t0; t < t1; ++t) gru_token<TO>(p, out, t, a.W, c, bz, bx, s);
}

LLMP_API int llmp_min_gru_chunk() { return SCAN_CHUNK; }

// scratch: float32 [3, R, chunks, W] when max_q_len > SCAN_CHUNK (chunks = ceil(max_q_len / SCAN_CHUNK)), else unused.
LLMP_API int llmp_min_gru(const float* p, const float* bias, const int* q_start, const int* slots, const int* positions,
                          float* state, void* out, int out_dtype, float* scratch, int R, int W, int max_q_len,
                          cudaStream_t stream) {
    if (R <= 0 || max_q_len <= 0) return 0;
    LLMP_REQUIRE(W > 0, "min_gru: bad width %d", W);
    GruArgs a;
    a.p = p; a.bias = bias; a.q_start = q_start; a.slots = slots; a.positions = positions; a.state = state;
    a.out = out; a.out_bf16 = out_dtype == LLMP_BF16; a.W = W;
    a.chunk_a = a.chunk_b = a.chunk_s = nullptr; a.chunks = 0;
    const int threads = 128;
    const int col_blocks = (W + threads - 1) / threads;
    if (max_q_len <= SCAN_CHUNK) {
        if (a.out_bf16) min_gru_serial_kernel<bf16><<<dim3(R, col_blocks), threads, 0, stream>>>(a);
        else min_gru_serial_kernel<float><<<dim3(R, col_blocks), threads, 0, stream>>>(a);
        return llmp_check_launch("min_gru");
    }
    LLMP_REQUIRE(scratch != nullptr, "min_gru: portions of more than %d tokens need scratch", SCAN_CHUNK);
    a.chunks = (max_q_len + SCAN_CHUNK - 1) / SCAN_CHUNK;
    LLMP_REQUIRE(a.chunks <= 65535 && col_blocks <= 65535, "min_gru: too many chunks %d", a.chunks);
    a.chunk_a = scratch;
    a.chunk_b = scratch + (size_t)R * a.chunks * W;
    a.chunk_s = scratch + 2 * (size_t)R * a.chunks * W;
    min_gru_chunk_kernel<<<dim3(R, a.chunks, col_blocks), threads, 0, stream>>>(a);
    min_gru_prefix_kernel<<<dim3(R, col_blocks), threads, 0, stream>>>(a);
    if (a.out_bf16) min_gru_apply_kernel<bf16><<<dim3(R, a.chunks, col_blocks), threads, 0, stream>>>(a);
    else min_gru_apply_kernel<float><<<dim3(R, a.chunks, col_blocks), threads, 0, stream>>>(a);
    return llmp_check_launch("min_gru (chunked)");
}
