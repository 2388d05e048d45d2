// Differential attention over bfloat16 pages on the tensor cores (mma.sync m16n8k16, float32 accumulate), with the
// arguments and result of llmp_diff_attention, for key sizes d and value sizes dv of 16, 32, 48, 64, 96 or 128.
//
// A block takes one tile of query rows of one request and one key/value head: DM_ROWS = 64 rows, a row being (token,
// query head of the group) with the head running fastest, so the key/value tile it streams serves all query heads of
// the group. A cached row is [key of map 1 | key of map 2 | value], so one copy brings both maps' keys and the values
// they share. Each of the four warps owns 16 rows and keeps, for both maps, the running softmax and the output in
// registers; a half tile of 32 keys is worked through for map 1, then for map 2, with the same value fragments. Keys
// are walked in tiles of 64 aligned to key 0 (the same operations for a row however the prompt was cut); tiles above
// the causal diagonal or below the window are skipped. At the end a row's two outputs are combined in registers:
// a1 - lambda a2, divided by its root mean square over the dv entries (a sum over the row's quad of lanes), scaled.
//
// The key/value tile has two buffers where two blocks of that size still fit an SM: the copy of the next tile runs under
// the products of this one.
//
// Steps of few rows over many keys (decoding): `segments` > 0 cuts the keys into segments of `segment_keys` (a multiple
// of the tile), every segment with blocks of its own that leave both maps' sums (maximum, sum, output; float32) in
// scratch and count themselves; the block of a tile that counts last adds the rows' segments in their order and does the
// combination (nobody waits, no second kernel; the counters are left at zero). When every tile is one token
// (`split`), its rows fit one warp's 16, and the four warps share a key tile instead: warp w takes half w / 2 of the
// tile's keys for map w % 2 and leaves sums of its own, so a segment has two sets of sums per map.
#include "common.cuh"

#define DM_ROWS 64
#define DM_KEYS 64
#define DM_THREADS 128

struct DiffMmaParams {
    const bf16* q;
    bf16* out;
    const bf16* pages;
    const int* block_tables;
    const int* q_start;
    const int* ctx_len;
    const int* tile_req;
    const int* tile_tok0;
    int* counters;                   // segments: one per (tile, kv head, chunk of heads), zero before and after a launch
    const int* positions;
    float* scratch;                  // segments: [segment][half of the tiles' keys, if split][token][head][map][dv + 2]
    long q_stride, out_stride;
    int table_stride;
    int nq, nkv, page_size, window;
    int heads_per_cta, tokens_per_cta, head_chunks, num_tiles;
    int segment_keys, segments, total_tokens, split, stages;
    float scale, lambda, eps, out_scale;
};

__device__ __forceinline__ void dm_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void dm_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void dm_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void dm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the special-function unit (relative error about 2^-22; the probabilities are rounded to bfloat16 anyway)
__device__ __forceinline__ float dm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ unsigned dm_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// One warp adds the sums that the segments left for row (token n, head h) at position `pos`, both maps, in the order of the
// segments' keys, and combines them: a1 - lambda a2, its norm, the store. The row's segments are those that hold a key it
// sees: from the one with its window's first key to the one with its own. Read past L1: other blocks wrote them.
__device__ __forceinline__ void dm_merge_row(const DiffMmaParams& p, int n, int h, int pos, int dv, int lane) {
    const int sets = p.split ? 2 : 1;
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int s_lo = lo / p.segment_keys, s_hi = pos / p.segment_keys;
    const int w = 2 * (dv + 2);
    const int first = s_lo * sets, count = (s_hi + 1) * sets - first;
    const float* base = p.scratch + (((size_t)first * p.total_tokens + n) * p.nq + h) * w;
    const size_t step = (size_t)p.total_tokens * p.nq * w;       // from one set of sums to the next
    // the maxima first (a lane per set), so that the sets can then be added without waiting for one another
    float m_all[2] = {-INFINITY, -INFINITY};
    for (int s = lane; s < count; s += 32) {
        m_all[0] = fmaxf(m_all[0], __ldcg(base + s * step));
        m_all[1] = fmaxf(m_all[1], __ldcg(base + s * step + dv + 2));
    }
    m_all[0] = warp_max(m_all[0]);
    m_all[1] = warp_max(m_all[1]);
    float acc[2][4], l_all[2] = {0.f, 0.f};
#pragma unroll
    for (int m = 0; m < 2; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
#pragma unroll 4
    for (int s = 0; s < count; ++s) {                            // in the order of the sets' keys
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const float* s2 = base + s * step + m * (dv + 2);
            const float a = exp2f(__ldcg(s2) - m_all[m]);        // log2 units, as the blocks keep them; 0 for a set without a visible key
            l_all[m] = fmaf(__ldcg(s2 + 1), a, l_all[m]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = lane + 32 * i;
                if (c < dv) acc[m][i] = fmaf(__ldcg(s2 + 2 + c), a, acc[m][i]);
            }
        }
    }
    const float i1 = 1.f / l_all[0], i2 = p.lambda / l_all[1];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = lane + 32 * i;
        acc[0][i] = c < dv ? acc[0][i] * i1 - acc[1][i] * i2 : 0.f;
        ss = fmaf(acc[0][i], acc[0][i], ss);
    }
    ss = warp_sum(ss);
    const float rn = rsqrtf(ss / (float)dv + p.eps) * p.out_scale;
    bf16* dst = p.out + (size_t)n * p.out_stride + (size_t)h * dv;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) dst[c] = __float2bfloat16_rn(acc[0][i] * rn);
    }
}

// D16: key size / 16; V16: value size / 16. With p.segments > 0 the keys are cut into segments (blockIdx.y) whose sums go
// to scratch.
template <int D16, int V16>
__global__ void __launch_bounds__(DM_THREADS, 2) diff_attention_mma_kernel(const DiffMmaParams p) {
    extern __shared__ __align__(16) unsigned char dm_smem[];
    const bool SEG = p.segments > 0;
    constexpr int D = D16 * 16, DV = V16 * 16;
    constexpr int QW = 2 * D, RS = 2 * D + DV;                   // a query row (both maps), a cached row
    constexpr int QSTRIDE = QW + 8, KSTRIDE = RS + 8;            // padded rows: conflict-free ldmatrix
    bf16* Qs = reinterpret_cast<bf16*>(dm_smem);                 // [DM_ROWS][QSTRIDE]
    bf16* ring = Qs + DM_ROWS * QSTRIDE;                         // [stages][DM_KEYS][KSTRIDE]
    constexpr int STAGE_ELEMS = DM_KEYS * KSTRIDE;
    __shared__ long long key_off[2][DM_KEYS];
    const bool split = p.split != 0;                             // four warps on the 16 rows of a one-token tile

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rw = split ? 0 : warp;                             // which 16 rows of the tile this warp works on
    const int per_tile = p.nkv * p.head_chunks;
    const int tile = p.num_tiles - 1 - (int)(blockIdx.x / (unsigned)per_tile);      // long tiles first
    const int in_tile = (int)(blockIdx.x % (unsigned)per_tile);
    const int r = p.tile_req[tile];
    const int tok0 = p.tile_tok0[tile];
    const int kvh = in_tile / p.head_chunks, chunk = in_tile % p.head_chunks;
    const int G = p.nq / p.nkv;
    const int hpc = p.heads_per_cta;
    const int head0 = chunk * hpc;
    int heads = G - head0;
    if (heads > hpc) heads = hpc;
    const int q_begin = p.q_start[r];
    const int q_len = p.q_start[r + 1] - q_begin;
    const int ctx = p.ctx_len[r];
    const int pos0 = ctx - q_len;
    int ntok = q_len - tok0;
    if (ntok > p.tokens_per_cta) ntok = p.tokens_per_cta;
    const int* table = p.block_tables + (size_t)r * p.table_stride;

    // keys this block needs: from the window start of its first token to the position of its last
    int hi = pos0 + tok0 + ntok - 1;                             // last key (inclusive)
    int lo = 0;
    if (p.window > 0) {
        lo = pos0 + tok0 - p.window + 1;
        if (lo < 0) lo = 0;
    }
    int tile_lo = (lo / DM_KEYS) * DM_KEYS;
    const int hi_tile = hi;                                      // the tile's last key, before a segment clips it
    if (SEG) {
        // segment s of a row holds the keys [s * segment_keys, (s + 1) * segment_keys) of its request, whatever the step
        const int s0 = (int)blockIdx.y * p.segment_keys;
        if (s0 > hi || s0 + p.segment_keys <= lo) return;        // nothing of this block's keys: the adding kernel skips it too
        if (tile_lo < s0) tile_lo = s0;
        if (hi > s0 + p.segment_keys - 1) hi = s0 + p.segment_keys - 1;
    }

    // query rows: row = token * hpc + head, both maps side by side
    constexpr int QVEC = QW / 8;
    for (int e = tid; e < DM_ROWS * QVEC; e += DM_THREADS) {
        const int row = e / QVEC, c = (e % QVEC) * 8;
        const int tl = row / hpc, h = row % hpc;
        const bool ok = tl < ntok && h < heads;
        const bf16* src = ok ? p.q + (size_t)(q_begin + tok0 + tl) * p.q_stride + (size_t)(kvh * G + head0 + h) * QW + c : p.q;
        dm_cp_async_16(Qs + row * QSTRIDE + c, src, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");

    constexpr int KVEC = RS / 8;
    auto issue_tile = [&](int j0, int buf) {
        if (tid < DM_KEYS) {
            const int j = j0 + tid;
            long long off = -1;
            if (j <= hi && j >= lo) {
                const int page = table[j / p.page_size];
                if (page >= 0) off = (long long)(((size_t)page * p.nkv + kvh) * p.page_size + (j % p.page_size)) * RS;
            }
            key_off[buf][tid] = off;
        }
        __syncthreads();
        bf16* dst = ring + (size_t)buf * STAGE_ELEMS;
        for (int e = tid; e < DM_KEYS * KVEC; e += DM_THREADS) {
            const int key = e / KVEC, c = (e % KVEC) * 8;
            const long long off = key_off[buf][key];
            const bool ok = off >= 0;
            dm_cp_async_16(dst + key * KSTRIDE + c, ok ? p.pages + off + c : p.pages, ok);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    // positions of this lane's two rows (row g and row g + 8 of the warp's 16); -1 for a row that does not exist
    int row_pos[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int row = rw * 16 + g + 8 * h2;
        const int tl = row / hpc, h = row % hpc;
        row_pos[h2] = (tl < ntok && h < heads) ? pos0 + tok0 + tl : -1;
    }

    float o[2][2 * V16][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int i = 0; i < 2 * V16; ++i) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.f;
    float m_run[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}};
    float l_run[2][2] = {{0.f, 0.f}, {0.f, 0.f}};

    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int warp_first_tok = (rw * 16) / hpc;
    const int warp_last_tok = (rw * 16 + 15) / hpc;
    const bool warp_has_rows = warp_first_tok < ntok;            // a warp without rows only helps with the copies
    const int warp_hi_pos = pos0 + tok0 + (warp_last_tok < ntok ? warp_last_tok : ntok - 1);
    const int warp_lo_pos = pos0 + tok0 + (warp_first_tok < ntok ? warp_first_tok : ntok - 1);
    const bf16* Qw = Qs + (size_t)(rw * 16 + (lane & 15)) * QSTRIDE + (lane >> 4) * 8;     // this lane's ldmatrix row of Q
    const bool two = p.stages == 2;
    if (two && tile_lo <= hi) issue_tile(tile_lo, 0);
    int buf = 0;
    for (int j0 = tile_lo; j0 <= hi; j0 += DM_KEYS) {
        if (two) {
            if (j0 + DM_KEYS <= hi) {
                issue_tile(j0 + DM_KEYS, buf ^ 1);               // its buffer was read last in the round before: see the barrier below
                asm volatile("cp.async.wait_group 1;\n" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            }
        } else {
            issue_tile(j0, 0);
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const bf16* KVs = ring + (size_t)buf * STAGE_ELEMS;
        if (warp_has_rows) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int jh = j0 + half * 32;
                if (split && half != (warp >> 1)) continue;      // another warp's keys
                if (jh > warp_hi_pos || jh > hi) continue;       // every row of this warp lies before these keys
                if (p.window > 0 && jh + 31 < warp_lo_pos - p.window + 1) continue;    // or sees none of them any more
                const bool need_mask = (jh + 31 > warp_lo_pos) || (jh + 31 > hi) || (p.window > 0 && jh < warp_hi_pos - p.window + 1);
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    if (split && m != (warp & 1)) continue;      // another warp's map
                    float s[4][4];
#pragma unroll
                    for (int nb = 0; nb < 4; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
                    for (int ks = 0; ks < D16; ++ks) {
                        unsigned qa[4];
                        dm_ldmatrix_x4(qa, Qw + m * D + ks * 16);
#pragma unroll
                        for (int nb = 0; nb < 4; nb += 2) {
                            unsigned kf[4];
                            dm_ldmatrix_x4(kf, KVs + (size_t)(half * 32 + (nb + (lane >> 4)) * 8 + (lane & 7)) * KSTRIDE + m * D + ks * 16 +
                                                   ((lane >> 3) & 1) * 8);
                            dm_mma(s[nb], qa, kf[0], kf[1]);
                            dm_mma(s[nb + 1], qa, kf[2], kf[3]);
                        }
                    }
                    float mx[2] = {-INFINITY, -INFINITY};
                    if (need_mask) {
#pragma unroll
                        for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const int j = jh + nb * 8 + 2 * t + (c & 1);
                                const int pos = row_pos[c >> 1];
                                bool ok = j <= pos && j <= hi;
                                if (p.window > 0 && j < pos - p.window + 1) ok = false;
                                if (!ok) s[nb][c] = -INFINITY;
                            }
                        }
                    }
#pragma unroll
                    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) mx[c >> 1] = fmaxf(mx[c >> 1], s[nb][c]);
                    }
                    // running max and sum live in units of log2 (exp(x * scale) = 2^(x * scale * log2 e))
                    float alpha[2], m_scaled[2];
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
                        mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
                        const float m_new = fmaxf(m_run[m][h2], mx[h2] * scale_log2);
                        alpha[h2] = (m_new > -INFINITY) ? dm_ex2(m_run[m][h2] - m_new) : 1.f;
                        m_run[m][h2] = m_new;
                        m_scaled[h2] = (m_new > -INFINITY) ? m_new : 0.f;     // a row without any key keeps p = 2^(-inf) = 0
                    }
                    float sum[2] = {0.f, 0.f};
#pragma unroll
                    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float pr = dm_ex2(fmaf(s[nb][c], scale_log2, -m_scaled[c >> 1]));
                            s[nb][c] = pr;
                            sum[c >> 1] += pr;
                        }
                    }
                    l_run[m][0] = l_run[m][0] * alpha[0] + sum[0];
                    l_run[m][1] = l_run[m][1] * alpha[1] + sum[1];
                    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                        for (int i = 0; i < 2 * V16; ++i) {
                            o[m][i][0] *= alpha[0]; o[m][i][1] *= alpha[0]; o[m][i][2] *= alpha[1]; o[m][i][3] *= alpha[1];
                        }
                    }
                    // O += P V, 16 keys per step
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        unsigned pa[4];
                        pa[0] = dm_pack(s[2 * kk][0], s[2 * kk][1]);
                        pa[1] = dm_pack(s[2 * kk][2], s[2 * kk][3]);
                        pa[2] = dm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                        pa[3] = dm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                        for (int nb2 = 0; nb2 < V16; ++nb2) {
                            unsigned v[4];
                            dm_ldmatrix_x4_trans(v, KVs + (size_t)(half * 32 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KSTRIDE + 2 * D +
                                                        nb2 * 16 + (lane >> 4) * 8);
                            dm_mma(o[m][nb2 * 2], pa, v[0], v[1]);
                            dm_mma(o[m][nb2 * 2 + 1], pa, v[2], v[3]);
                        }
                    }
                }
            }
        }
        __syncthreads();                                         // the tile's buffer may be overwritten now
        if (two) buf ^= 1;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");       // the query copy, where no key tile followed it

#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            l_run[m][h2] += __shfl_xor_sync(0xffffffffu, l_run[m][h2], 1);
            l_run[m][h2] += __shfl_xor_sync(0xffffffffu, l_run[m][h2], 2);
        }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int row = rw * 16 + g + 8 * h2;
        const int tl = row / hpc, h = row % hpc;
        const bool exists = row_pos[h2] >= 0;
        if (SEG) {
            if (!exists) continue;
            const size_t set = split ? (size_t)blockIdx.y * 2 + (warp >> 1) : (size_t)blockIdx.y;
            float* dst = p.scratch + ((set * p.total_tokens + (q_begin + tok0 + tl)) * p.nq + (kvh * G + head0 + h)) * (2 * (DV + 2));
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                if (split && m != (warp & 1)) continue;
                float* d2 = dst + m * (DV + 2);
                if (t == 0) {
                    d2[0] = m_run[m][h2];
                    d2[1] = l_run[m][h2];
                }
#pragma unroll
                for (int nb = 0; nb < 2 * V16; ++nb) {
                    d2[2 + nb * 8 + 2 * t] = o[m][nb][2 * h2];
                    d2[2 + nb * 8 + 2 * t + 1] = o[m][nb][2 * h2 + 1];
                }
            }
            continue;
        }
        const float i1 = l_run[0][h2] > 0.f ? 1.f / l_run[0][h2] : 0.f;
        const float i2 = l_run[1][h2] > 0.f ? p.lambda / l_run[1][h2] : 0.f;
        float ss = 0.f;
#pragma unroll
        for (int nb = 0; nb < 2 * V16; ++nb) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float v = o[0][nb][2 * h2 + c] * i1 - o[1][nb][2 * h2 + c] * i2;
                o[0][nb][2 * h2 + c] = v;
                ss = fmaf(v, v, ss);
            }
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);               // all lanes take part: no lane has left the loop
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (!exists) continue;
        const float rn = rsqrtf(ss / (float)DV + p.eps) * p.out_scale;
        bf16* dst = p.out + (size_t)(q_begin + tok0 + tl) * p.out_stride + (size_t)(kvh * G + head0 + h) * DV + 2 * t;
#pragma unroll
        for (int nb = 0; nb < 2 * V16; ++nb)
            *reinterpret_cast<unsigned*>(dst + nb * 8) = dm_pack(o[0][nb][2 * h2] * rn, o[0][nb][2 * h2 + 1] * rn);
    }
    if (SEG) {
        // every block of this tile whose segment holds one of the tile's keys counts itself once its sums are out; the one
        // that counts last adds them up
        __shared__ int is_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int needed = hi_tile / p.segment_keys - lo / p.segment_keys + 1;
            is_last = atomicAdd(&p.counters[blockIdx.x], 1) == needed - 1;
            if (is_last) p.counters[blockIdx.x] = 0;
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            for (int row = warp; row < ntok * heads; row += DM_THREADS / 32) {
                const int tl = row / heads, h = row % heads;
                dm_merge_row(p, q_begin + tok0 + tl, kvh * G + head0 + h, pos0 + tok0 + tl, DV, lane);
            }
        }
    }
}

// Sizes the kernel is instantiated for: 16, 32, 48, 64, 96, 128 for keys and for values.
static bool dm_size_served(int n) { return n == 16 || n == 32 || n == 48 || n == 64 || n == 96 || n == 128; }

LLMP_API int llmp_diff_mma_supports(int d, int dv, int page_size) {
    (void)page_size;
    return dm_size_served(d) && dm_size_served(dv);
}

// Query tokens per block for a group size: 64 rows of (token, head).
LLMP_API int llmp_diff_mma_tokens_per_tile(int nq, int nkv) {
    const int G = nq / nkv;
    const int hpc = G < 16 ? G : 16;
    return DM_ROWS / hpc;
}

template <int D16, int V16>
static int launch_diff_mma(const DiffMmaParams& p, unsigned grid, cudaStream_t stream) {
    const size_t q_bytes = sizeof(bf16) * (size_t)DM_ROWS * (2 * D16 * 16 + 8);
    const size_t stage = sizeof(bf16) * (size_t)DM_KEYS * (2 * D16 * 16 + V16 * 16 + 8);
    DiffMmaParams q = p;
    q.stages = q_bytes + 2 * stage <= 110 * 1024 ? 2 : 1;        // two buffers where two blocks of that size still share an SM
    const size_t smem = q_bytes + q.stages * stage;
    LLMP_ALLOW_SMEM((diff_attention_mma_kernel<D16, V16>), smem);
    diff_attention_mma_kernel<D16, V16><<<dim3(grid, p.segments > 0 ? p.segments : 1), DM_THREADS, smem, stream>>>(q);
    return 0;
}

LLMP_API int llmp_diff_attention_mma(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                                     const int* block_tables, int table_stride, const int* q_start, const int* ctx_len,
                                     const int* positions, const int* tile_req, const int* tile_tok0, int num_tiles, int total_tokens,
                                     int nq, int nkv, int d, int dv, int page_size, int window, float scale, float lambda, float eps,
                                     float out_scale, int segment_keys, int segments, int split, float* scratch, int* counters,
                                     cudaStream_t stream) {
    if (num_tiles <= 0 || total_tokens <= 0) return 0;
    LLMP_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && llmp_diff_mma_supports(d, dv, page_size) && page_size > 0 && window >= 0,
                 "diff_attention_mma: sizes heads=%d kv_heads=%d dim=%d vdim=%d are not served", nq, nkv, d, dv);
    LLMP_REQUIRE(segments == 0 || (scratch && counters && segment_keys > 0 && segment_keys % DM_KEYS == 0 && segments <= 65535),
                 "diff_attention_mma: segments need scratch, counters and a length that is a multiple of %d", DM_KEYS);
    DiffMmaParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.pages = (const bf16*)pages; p.block_tables = block_tables;
    p.q_start = q_start; p.ctx_len = ctx_len; p.tile_req = tile_req; p.tile_tok0 = tile_tok0; p.scratch = scratch;
    p.counters = counters; p.positions = positions;
    p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv;
    p.page_size = page_size; p.window = window; p.scale = scale; p.lambda = lambda; p.eps = eps; p.out_scale = out_scale;
    const int G = nq / nkv;
    p.heads_per_cta = G < 16 ? G : 16;
    p.tokens_per_cta = DM_ROWS / p.heads_per_cta;
    p.head_chunks = (G + p.heads_per_cta - 1) / p.heads_per_cta;
    p.num_tiles = num_tiles;
    p.segment_keys = segment_keys; p.segments = segments; p.total_tokens = total_tokens;
    p.split = (split && segments > 0) ? 1 : 0; p.stages = 1;
    LLMP_REQUIRE(!p.split || num_tiles == total_tokens, "diff_attention_mma: warps share a tile's keys only in steps of one token a request");
    LLMP_REQUIRE((long)num_tiles * nkv * p.head_chunks < (1L << 31), "diff_attention_mma: too many tiles");
    LLMP_REQUIRE((q_stride % 8) == 0 && (out_stride % 2) == 0 && ((size_t)q % 16) == 0 && ((size_t)pages % 16) == 0,
                 "diff_attention_mma: query rows must be 16-byte aligned");
    const unsigned grid = (unsigned)(num_tiles * nkv * p.head_chunks);
    int rc = 1;
#define DM_V(DD, VV) case VV: rc = launch_diff_mma<DD, VV>(p, grid, stream); break;
#define DM_D(DD)                                                                              \
    case DD:                                                                                  \
        switch (dv / 16) { DM_V(DD, 1) DM_V(DD, 2) DM_V(DD, 3) DM_V(DD, 4) DM_V(DD, 6) DM_V(DD, 8) } \
        break;
    switch (d / 16) { DM_D(1) DM_D(2) DM_D(3) DM_D(4) DM_D(6) DM_D(8) }
#undef DM_D
#undef DM_V
    if (rc) return rc;
    return llmp_check_launch("diff_attention_mma");
}
