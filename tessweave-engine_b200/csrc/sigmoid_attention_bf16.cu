// Sigmoid attention with folded queries on tensor cores (bfloat16, mma.sync.m16n8k16, fp32 scores and sums),
// one compiled library per head size (-DTW_HEAD_DIM, a multiple of 16 up to 256).
//
// What the kernels compute is described at the top of sigmoid_attention.cu: after the fold a head is an
// attention head whose query has G * D values and meets the keys of all G key/value heads of a position,
//   s = sum_c qf_c . k_c(j),   w = sigmoid(s + b_h) for visible j,   o = sum_j w v_c(h)(j),
// no maximum, no normalisation, so nothing is rescaled and partial sums over slices of keys just add.
//
// Keys and values reach shared memory in *chunks*: 64 keys of one key/value head, rows padded by 16 bytes
// (conflict-free ldmatrix for every head size), through a ring of four cp.async stages.  A tile of 64 keys is
// the chunks K_0 .. K_{G-1} (scores accumulate over them) followed by the value chunk(s).  Keys a row must not
// see get weight 0, and their rows are zero-filled in shared memory, so nothing of a page that was freed or
// never written reaches a sum.
//
//   prompt portions   block = 64 or 128 consecutive tokens of one request x one head; warp w owns rows 16w .. 16w + 15
//   single tokens     block = one request x 16 heads x one slice of the keys; warp w owns keys 16w .. 16w + 15 of
//                     every tile; heads of different key/value groups take their values from different chunks
//                     (the weights of the other rows are zeroed for that product); the four warps' sums meet in
//                     shared memory, the slices' sums in scratch memory, added in slice order by a second kernel
//                     that also applies the output gate.
#include "attention_common.cuh"

#ifndef TW_HEAD_DIM
#define TW_HEAD_DIM 128
#endif

using namespace tw_attn;

namespace {

constexpr int D = TW_HEAD_DIM;
constexpr int BN = 64;                      // keys per tile
constexpr int KSTR = D + 8;                 // padded row of a chunk (elements)
constexpr int CHUNK = BN * KSTR;            // elements per stage
constexpr int NSTAGE = 4;                   // three chunks are under way while one is consumed
constexpr int THREADS = 128;             // of the single-token kernel; the prompt kernel has 32 x its warps
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 up to 256");

__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// Where the 16-byte pieces a thread copies for a tile of 64 keys come from: the page and the place inside it
// are the same for every key/value head and for keys and values, so they are looked up once per tile and a chunk
// costs a thread a few additions per piece.  Keys outside [j_lo, j_hi) get -1: their rows are zero-filled.
template <int NT_THREADS>
struct TileRows {
    static constexpr int CPR = D / 8;                                   // 16-byte pieces per row
    static constexpr int NI = (BN * CPR + NT_THREADS - 1) / NT_THREADS; // pieces per thread
    long long off[NI];

    __device__ __forceinline__ void look_up(const int* __restrict__ table, int table_stride, int j0, int j_lo, int j_hi,
                                            int G, int P, int num_pages, int* status) {
#pragma unroll
        for (int k = 0; k < NI; ++k) {
            const int i = threadIdx.x + k * NT_THREADS;
            const int r = i / CPR, piece = i - r * CPR;
            const int j = j0 + r;
            off[k] = -1;
            if (i < BN * CPR && j >= j_lo && j < j_hi) {
                const int blk = j / P;
                const int page = blk < table_stride ? table[blk] : -1;
                if (page < 0 || page >= num_pages) {
                    if (piece == 0) atomicOr(status, TW_ERR_PAGE);
                } else {
                    off[k] = ((long long)page * G * P + (j - blk * P)) * D + piece * 8;
                }
            }
        }
    }

    // the chunk of key/value head c into one stage
    __device__ __forceinline__ void load(bf16* dst, const bf16* __restrict__ cache, int c, int P) const {
        const long long head = (long long)c * P * D;
#pragma unroll
        for (int k = 0; k < NI; ++k) {
            const int i = threadIdx.x + k * NT_THREADS;
            if (i < BN * CPR) {
                const int r = i / CPR, piece = i - r * CPR;
                const bool live = off[k] >= 0;
                cp_async16(dst + r * KSTR + piece * 8, live ? cache + off[k] + head : cache, live ? 16 : 0);
            }
        }
    }
};

// S[nt] += A(16 rows of q, columns c * D ..) . K(keys key0 + 8 nt ..)^T for NT tiles of eight keys (NT even).
template <int NT>
__device__ __forceinline__ void scores_chunk(float (&S)[NT][4], const bf16* qs, int qstr, int qrow0, int c,
                                             const bf16* ks, int key0, int lane) {
    const int a_row = qrow0 + (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_key = key0 + (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int kd = 0; kd < D / 16; ++kd) {
        uint32_t a[4];
        ldmatrix_x4(a, qs + (size_t)a_row * qstr + c * D + kd * 16 + a_col);
#pragma unroll
        for (int p = 0; p < NT / 2; ++p) {
            uint32_t b[4];
            ldmatrix_x4(b, ks + (b_key + p * 16) * KSTR + kd * 16 + b_col);
            mma_bf16(S[2 * p], a, b[0], b[1]);
            mma_bf16(S[2 * p + 1], a, b[2], b[3]);
        }
    }
}

// O += P(16 rows x 16 keys) . V(keys key0 .. key0 + 15), all D columns.
__device__ __forceinline__ void values_step(float (&O)[D / 8][4], const uint32_t (&pa)[4], const bf16* vs, int key0,
                                            int lane) {
    const int v_key = key0 + (lane & 7) + ((lane >> 3) & 1) * 8, v_col = (lane >> 4) * 8;
#pragma unroll
    for (int nd = 0; nd < D / 16; ++nd) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vs + v_key * KSTR + nd * 16 + v_col);
        mma_bf16(O[2 * nd], pa, b[0], b[1]);
        mma_bf16(O[2 * nd + 1], pa, b[2], b[3]);
    }
}

// The same for MT tiles of sixteen rows against ONE slab of sixteen keys (the single-token kernel): a fragment of
// the keys is loaded once and meets every row tile, and the products of different row tiles do not wait for one another.
template <int MT>
__device__ __forceinline__ void scores_slab(float (&S)[MT][2][4], const bf16* qs, int qstr, int c, const bf16* ks, int key0,
                                            int lane, int live_tiles) {
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;
    const int b_key = key0 + (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int kd = 0; kd < D / 16; ++kd) {
        uint32_t b[4];
        ldmatrix_x4(b, ks + b_key * KSTR + kd * 16 + b_col);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < live_tiles) {
                uint32_t a[4];
                ldmatrix_x4(a, qs + (size_t)(m * 16 + a_row) * qstr + c * D + kd * 16 + a_col);
                mma_bf16(S[m][0], a, b[0], b[1]);
                mma_bf16(S[m][1], a, b[2], b[3]);
            }
        }
    }
}

// O[m] += P[m](16 rows x 16 keys) . V(keys key0 .. key0 + 15) for the row tiles whose bit is set in `use`.
template <int MT>
__device__ __forceinline__ void values_slab(float (&O)[MT][D / 8][4], const uint32_t (&pa)[MT][4], const bf16* vs, int key0,
                                            int lane, int use) {
    const int v_key = key0 + (lane & 7) + ((lane >> 3) & 1) * 8, v_col = (lane >> 4) * 8;
#pragma unroll
    for (int nd = 0; nd < D / 16; ++nd) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vs + v_key * KSTR + nd * 16 + v_col);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (use & (1 << m)) {
                mma_bf16(O[m][2 * nd], pa[m], b[0], b[1]);
                mma_bf16(O[m][2 * nd + 1], pa[m], b[2], b[3]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Prompt portions.
// ---------------------------------------------------------------------------------------
template <int WARPS>
__global__ void __launch_bounds__(32 * WARPS)
sigattn_prefill_kernel(bf16* __restrict__ out, int out_stride, const bf16* __restrict__ qf,
                       const float* __restrict__ bias, const bf16* __restrict__ gate, int gate_stride,
                       const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                       const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                       const int* __restrict__ block_table, int table_stride, const bf16* __restrict__ k_cache,
                       const bf16* __restrict__ v_cache, int H, int G, int P, int num_pages, int window,
                       int skip_singles, int* status) {
    constexpr int BM = 16 * WARPS;          // token rows of a block
    extern __shared__ __align__(16) unsigned char smem_raw[];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int s = blockIdx.z, h = blockIdx.y, tile = blockIdx.x;
    const int q_len = seq_q_len[s];
    if (tile * BM >= q_len || (skip_singles && q_len == 1)) return;
    const int q_start = seq_q_start[s], kv_len = seq_kv_len[s];
    const int rows_valid = min(BM, q_len - tile * BM);
    const int row0 = q_start + tile * BM;                 // first token row of the tile
    const int pos0 = kv_len - q_len + tile * BM;          // its position
    const int j_hi = pos0 + rows_valid;                   // keys below this are seen by some row
    const int j_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int t0 = j_lo / BN, ntiles = (j_hi - 1) / BN - t0 + 1;
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;
    const int KW = G * D, QSTR = KW + 8;
    const int kvh = h / (H / G);
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* ring = qs + BM * QSTR;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // the folded queries of the tile (rows past the portion's end are zero)
    {
        const int pieces = KW / 8;
        for (int i = threadIdx.x; i < BM * pieces; i += 32 * WARPS) {
            const int r = i / pieces, piece = i - r * pieces;
            const bool live = r < rows_valid;
            const bf16* src = live ? qf + ((size_t)(row0 + r) * H + h) * KW + piece * 8 : qf;
            cp_async16(qs + r * QSTR + piece * 8, src, live ? 16 : 0);
        }
    }
    const int per_tile = G + 1;
    const int nchunks = ntiles * per_tile;
    TileRows<32 * WARPS> rows;
    auto issue = [&](int n) {
        if (n < nchunks) {
            const int t = n / per_tile, k = n - t * per_tile;
            bf16* dst = ring + (n % NSTAGE) * CHUNK;
            if (k == 0) rows.look_up(table, table_stride, (t0 + t) * BN, j_lo, j_hi, G, P, num_pages, status);
            if (k < G) rows.load(dst, k_cache, k, P);
            else rows.load(dst, v_cache, kvh, P);
        }
        cp_async_commit();
    };
    for (int n = 0; n < NSTAGE - 1; ++n) issue(n);
    float S[8][4], O[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f; }
    const float b = bias ? bias[h] : 0.f;
    const int g = lane >> 2, tq = lane & 3;
    for (int n = 0; n < nchunks; ++n) {
        // chunk n has landed for every thread, and every warp is done with chunk n - 1, whose stage is filled next
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();
        issue(n + NSTAGE - 1);
        const int t = n / per_tile, k = n - t * per_tile;
        const bf16* stage = ring + (n % NSTAGE) * CHUNK;
        if (k < G) {
            if (k == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) { S[i][0] = S[i][1] = S[i][2] = S[i][3] = 0.f; }
            }
            scores_chunk<8>(S, qs, QSTR, warp * 16, k, stage, 0, lane);
        } else {
            const int jbase = (t0 + t) * BN;
            const int pos_a = pos0 + warp * 16 + g, pos_b = pos_a + 8;
            const bool live_a = warp * 16 + g < rows_valid, live_b = warp * 16 + g + 8 < rows_valid;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pa[4];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int nt = 2 * kk + half;
                    const int j = jbase + nt * 8 + 2 * tq;
                    float w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int je = j + (e & 1);
                        const int pos = (e & 2) ? pos_b : pos_a;
                        const bool ok = ((e & 2) ? live_b : live_a) && je <= pos && (window <= 0 || je > pos - window);
                        w[e] = ok ? sigmoid_fast(S[nt][e] + b) : 0.f;
                    }
                    pa[half * 2] = pack_bf16(w[0], w[1]);
                    pa[half * 2 + 1] = pack_bf16(w[2], w[3]);
                }
                values_step(O, pa, stage, kk * 16, lane);
            }
        }
    }
    // the output gate, then rows g and g + 8 of the warp's sixteen
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + g + half * 8;
        if (r >= rows_valid) continue;
        bf16* orow = out + (size_t)(row0 + r) * out_stride + h * D;
        const bf16* grow = gate ? gate + (size_t)(row0 + r) * gate_stride + h * D : nullptr;
#pragma unroll
        for (int nd = 0; nd < D / 8; ++nd) {
            const int col = nd * 8 + 2 * tq;
            float x = O[nd][half * 2], y = O[nd][half * 2 + 1];
            if (grow) {
                const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(grow + col));
                x *= sigmoid_fast(gv.x);
                y *= sigmoid_fast(gv.y);
            }
            *reinterpret_cast<__nv_bfloat162*>(orow + col) = __floats2bfloat162_rn(x, y);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Single tokens, keys cut into slices.  partial: [request][slice][head][D] fp32.
// ---------------------------------------------------------------------------------------
template <int MT>        // tiles of 16 heads a block serves: all heads of a request up to 16 * MT, so the keys are read once
__global__ void __launch_bounds__(THREADS)
sigattn_decode_kernel(float* __restrict__ partial, const bf16* __restrict__ qf, const float* __restrict__ bias,
                      const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                      const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                      const int* __restrict__ block_table, int table_stride, const bf16* __restrict__ k_cache,
                      const bf16* __restrict__ v_cache, int H, int G, int P, int num_pages, int window, int nsplit,
                      int* status) {
    constexpr int HB = 16 * MT;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int sp = blockIdx.x, ht = blockIdx.y, s = blockIdx.z;
    if (seq_q_len[s] != 1) return;
    const int row = seq_q_start[s], kv_len = seq_kv_len[s];
    const int pos = kv_len - 1;
    const int j_hi = kv_len, j_lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int t0 = j_lo / BN, ntiles_all = (j_hi - 1) / BN - t0 + 1;
    const int per = (ntiles_all + nsplit - 1) / nsplit;
    const int t_first = t0 + sp * per, ntiles = max(0, min(per, ntiles_all - sp * per));
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;
    const int KW = G * D, QSTR = KW + 8;
    const int group = H / G;
    const int h0 = ht * HB, heads = min(HB, H - h0);
    const int c_lo = h0 / group, c_hi = (h0 + heads - 1) / group;       // key/value heads this block's values come from
    const int nv = c_hi - c_lo + 1;
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* ring = qs + HB * QSTR;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {
        const int pieces = KW / 8;
        for (int i = threadIdx.x; i < HB * pieces; i += THREADS) {
            const int r = i / pieces, piece = i - r * pieces;
            const bool live = r < heads;
            const bf16* src = live ? qf + ((size_t)row * H + h0 + r) * KW + piece * 8 : qf;
            cp_async16(qs + r * QSTR + piece * 8, src, live ? 16 : 0);
        }
    }
    const int per_tile = G + nv;
    const int nchunks = ntiles * per_tile;
    TileRows<THREADS> rows;
    auto issue = [&](int n) {
        if (n < nchunks) {
            const int t = n / per_tile, k = n - t * per_tile;
            bf16* dst = ring + (n % NSTAGE) * CHUNK;
            if (k == 0) rows.look_up(table, table_stride, (t_first + t) * BN, j_lo, j_hi, G, P, num_pages, status);
            if (k < G) rows.load(dst, k_cache, k, P);
            else rows.load(dst, v_cache, c_lo + (k - G), P);
        }
        cp_async_commit();
    };
    for (int n = 0; n < NSTAGE - 1; ++n) issue(n);
    float S[MT][2][4], O[MT][D / 8][4], w[MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { O[m][i][0] = O[m][i][1] = O[m][i][2] = O[m][i][3] = 0.f; }
    }
    const int g = lane >> 2, tq = lane & 3;
    float b_a[MT], b_b[MT];
    int c_a[MT], c_b[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const int head_a = h0 + m * 16 + g, head_b = head_a + 8;
        b_a[m] = (bias && head_a < H) ? bias[head_a] : 0.f;
        b_b[m] = (bias && head_b < H) ? bias[head_b] : 0.f;
        c_a[m] = head_a < H ? head_a / group : -1;
        c_b[m] = head_b < H ? head_b / group : -1;
    }
    for (int n = 0; n < nchunks; ++n) {
        // chunk n has landed for every thread, and every warp is done with chunk n - 1, whose stage is filled next
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();
        issue(n + NSTAGE - 1);
        const int t = n / per_tile, k = n - t * per_tile;
        const bf16* stage = ring + (n % NSTAGE) * CHUNK;
        const int live_tiles = (heads + 15) >> 4;
        if (k < G) {
            if (k == 0) {
#pragma unroll
                for (int m = 0; m < MT; ++m) {
#pragma unroll
                    for (int i = 0; i < 2; ++i) { S[m][i][0] = S[m][i][1] = S[m][i][2] = S[m][i][3] = 0.f; }
                }
            }
            scores_slab<MT>(S, qs, QSTR, k, stage, warp * 16, lane, live_tiles);
        } else {
            const int c = c_lo + (k - G);
            if (k == G) {
                const int jbase = (t_first + t) * BN + warp * 16;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int je = jbase + nt * 8 + 2 * tq + (e & 1);
                            const bool ok = m < live_tiles && je >= j_lo && je < j_hi && ((e & 2) ? c_b[m] : c_a[m]) >= 0;
                            w[m][nt][e] = ok ? sigmoid_fast(S[m][nt][e] + ((e & 2) ? b_b[m] : b_a[m])) : 0.f;
                        }
                    }
                }
            }
            uint32_t pa[MT][4];
            int use = 0;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                // does any head of this tile of sixteen take its values from key/value head c?
                const int m_lo = (h0 + m * 16) / group, m_hi = (min(H, h0 + m * 16 + 16) - 1) / group;
                if (m < live_tiles && c >= m_lo && c <= m_hi) use |= 1 << m;
                const bool use_a = c_a[m] == c, use_b = c_b[m] == c;
                pa[m][0] = use_a ? pack_bf16(w[m][0][0], w[m][0][1]) : 0u;
                pa[m][1] = use_b ? pack_bf16(w[m][0][2], w[m][0][3]) : 0u;
                pa[m][2] = use_a ? pack_bf16(w[m][1][0], w[m][1][1]) : 0u;
                pa[m][3] = use_b ? pack_bf16(w[m][1][2], w[m][1][3]) : 0u;
            }
            values_slab<MT>(O, pa, stage, warp * 16, lane, use);
        }
    }
    // the four warps' sums meet in shared memory (the ring is free now), in warp order, one tile of heads at a time
    cp_async_wait<0>();
    __syncthreads();
    float* sums = reinterpret_cast<float*>(ring);          // [4][16][D]
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        if (m * 16 >= heads) continue;
#pragma unroll
        for (int nd = 0; nd < D / 8; ++nd) {
            const int col = nd * 8 + 2 * tq;
            *reinterpret_cast<float2*>(sums + ((size_t)warp * 16 + g) * D + col) = make_float2(O[m][nd][0], O[m][nd][1]);
            *reinterpret_cast<float2*>(sums + ((size_t)warp * 16 + g + 8) * D + col) = make_float2(O[m][nd][2], O[m][nd][3]);
        }
        __syncthreads();
        const int live = min(16, heads - m * 16);
        float* dst = partial + (((size_t)s * nsplit + sp) * H + h0 + m * 16) * D;
        for (int i = threadIdx.x; i < live * D; i += THREADS) {
            dst[i] = ((sums[i] + sums[16 * D + i]) + sums[2 * 16 * D + i]) + sums[3 * 16 * D + i];
        }
        __syncthreads();
    }
}

// out[token, h, :] = bf16((sum over slices, in slice order) * sigmoid(gate)).
__global__ void sigattn_decode_merge_kernel(bf16* __restrict__ out, int out_stride, const float* __restrict__ partial,
                                            const bf16* __restrict__ gate, int gate_stride,
                                            const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                                            int H, int nsplit) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int s = blockIdx.y;
    if (seq_q_len[s] != 1) return;
    const int row = seq_q_start[s];
    const int width = H * D;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < width; i += gridDim.x * blockDim.x) {
        const float* src = partial + (size_t)s * nsplit * width + i;
        float acc = 0.f;
        int sp = 0;
        for (; sp + 8 <= nsplit; sp += 8) {              // eight loads under way, added in slice order
            float v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = src[(size_t)(sp + k) * width];
#pragma unroll
            for (int k = 0; k < 8; ++k) acc += v[k];
        }
        for (; sp < nsplit; ++sp) acc += src[(size_t)sp * width];
        if (gate) acc *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[(size_t)row * gate_stride + i])));
        out[(size_t)row * out_stride + i] = __float2bfloat16_rn(acc);
    }
}

}  // namespace

static size_t ring_bytes() { return (size_t)NSTAGE * CHUNK * sizeof(bf16); }

TW_EXPORT int tw_sigattn_head_dim() { return D; }

// Shared memory a launch needs, for the caller to decide whether the shape fits (227 KB per block).
TW_EXPORT long tw_sigattn_prefill_smem(int G, int rows) { return (long)((size_t)rows * (G * D + 8) * sizeof(bf16) + ring_bytes()); }
TW_EXPORT long tw_sigattn_decode_smem(int G, int heads_per_block) {
    return (long)((size_t)heads_per_block * (G * D + 8) * sizeof(bf16) + ring_bytes());     // the ring also holds the warps' sums
}

TW_EXPORT int tw_sigattn_prefill(void* out, int out_stride, const void* qf, const float* bias, const void* gate,
                                 int gate_stride, const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len,
                                 const int* seq_slot, const int* block_table, int table_stride, const void* k_cache,
                                 const void* v_cache, int n_seqs, int max_q_len, int H, int G, int page_size,
                                 int num_pages, int window, int skip_singles, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (G <= 0 || H % G) return (int)cudaErrorInvalidValue;
    // 128-row blocks (eight warps) read every chunk for twice the rows; they pay where portions are long and fit
    const bool wide = max_q_len >= 128 && (size_t)tw_sigattn_prefill_smem(G, 128) <= 227 * 1024;
    const int rows = wide ? 128 : 64;
    const size_t smem = (size_t)tw_sigattn_prefill_smem(G, rows);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    auto kernel = wide ? sigattn_prefill_kernel<8> : sigattn_prefill_kernel<4>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const dim3 grid((max_q_len + rows - 1) / rows, H, n_seqs);
    return tw_launch(kernel, grid, dim3(rows * 2), smem, stream, 1, (bf16*)out, out_stride, (const bf16*)qf,
                     bias, (const bf16*)gate, gate_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table,
                     table_stride, (const bf16*)k_cache, (const bf16*)v_cache, H, G, page_size, num_pages, window,
                     skip_singles, status);
}

TW_EXPORT int tw_sigattn_decode(void* out, int out_stride, float* partial, const void* qf, const float* bias,
                                const void* gate, int gate_stride, const int* seq_q_start, const int* seq_q_len,
                                const int* seq_kv_len, const int* seq_slot, const int* block_table, int table_stride,
                                const void* k_cache, const void* v_cache, int n_seqs, int H, int G, int page_size,
                                int num_pages, int window, int nsplit, int heads_per_block, int* status, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (G <= 0 || H % G || nsplit <= 0) return (int)cudaErrorInvalidValue;
    // a block serves 32 heads where there are more than 16 (the keys are then read once for all of them)
    const bool two = H > 16 && heads_per_block != 16 && (size_t)tw_sigattn_decode_smem(G, 32) <= 227 * 1024;
    const int hb = two ? 32 : 16;
    const size_t smem = (size_t)tw_sigattn_decode_smem(G, hb);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    auto kernel = two ? sigattn_decode_kernel<2> : sigattn_decode_kernel<1>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const dim3 grid(nsplit, (H + hb - 1) / hb, n_seqs);
    int code = tw_launch(kernel, grid, dim3(THREADS), smem, stream, 1, partial, (const bf16*)qf, bias,
                         seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, table_stride, (const bf16*)k_cache,
                         (const bf16*)v_cache, H, G, page_size, num_pages, window, nsplit, status);
    if (code != 0) return code;
    const int width = H * D;
    const dim3 mgrid((width + 255) / 256, n_seqs);
    return tw_launch(sigattn_decode_merge_kernel, mgrid, dim3(256), 0, stream, 1, (bf16*)out, out_stride,
                     (const float*)partial, (const bf16*)gate, gate_stride, seq_q_start, seq_q_len, H, nsplit);
}
