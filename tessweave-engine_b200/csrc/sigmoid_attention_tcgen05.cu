// Sigmoid attention with folded queries for prompt portions on the 5th-generation tensor cores, for one head
// size (compile with -DTW_HEAD_DIM=64 or 128).  What is computed: see the top of sigmoid_attention.cu.
//
// A block serves 128 rows of one (request, key/value head c), a row being a (token, query head of c's group)
// pair, and walks the request's keys in tiles of 128 (or 64: -DTW_SIG_KEY_TILE).  Per key tile:
//     S = sum over key/value heads g of  Qf_g K_g^T     tcgen05.mma accumulating over the G chunks of the folded
//                                                       query (K-major, shared memory); S (fp32) in tensor memory
//     P = sigmoid(S + b_h), 0 where a key is not seen    four warps, one row (one TMEM lane) per thread: tcgen05.ld,
//                                                       P rounded to bf16 and stored over S (tcgen05.st)
//     O += P V_c                                         tcgen05.mma with P as the operand in tensor memory and V read
//                                                       "MN-major" straight from the page layout [key][d]
// Nothing carries over from one key tile to the next (no maximum, no normalisation), so S has two buffers in
// tensor memory and two groups of four warps take the even and the odd key tiles: the tensor cores form S of
// tile i + 1 while the sigmoids of tile i are evaluated.  Keys and values travel by TMA (cp.async.bulk.tensor.2d,
// no multicast), one box per page and 64 columns of d; the key chunks of all G key/value heads go through one
// ring, the values through another.  One warp issues the copies, one thread every MMA.
//
// Value rows beyond the request's last key are zeroed in shared memory, so stale page contents cannot reach a
// product.  Every wait on an mbarrier is bounded; a wait that runs out sets TW_ERR_WAIT in the status word,
// every role stops, the block waits (bounded) for its copies in flight, frees its tensor memory and returns.
#include "tcgen05.cuh"

#ifndef TW_HEAD_DIM
#define TW_HEAD_DIM 128
#endif
#ifndef TW_SIG_KEY_TILE
#define TW_SIG_KEY_TILE 128
#endif

namespace {

using namespace tc5;

constexpr int D = TW_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 sigmoid attention is built for head sizes 64 and 128");

constexpr int BM = 128;                       // rows of a block = TMEM lanes
constexpr int BN = TW_SIG_KEY_TILE;           // keys per tile (64 or 128): small chunks make the rings beside the folded queries deep
static_assert(BN == 64 || BN == 128, "key tiles of 64 or 128");
constexpr int KB = D / 64;                    // 64-column blocks of a row of q, k or v
constexpr int BLK = BM * 128;                 // bytes of a [128 rows][64 columns] swizzled block (the queries)
constexpr int KBLK = BN * 128;                // bytes of a [64 keys][64 columns] swizzled block (keys and values)
constexpr int CHUNK_BYTES = KB * KBLK;        // 64 keys of one key/value head
constexpr int MAX_K_STAGES = 12, MAX_V_STAGES = 3;
constexpr int BARRIER_BYTES = 512;            // 2 x 12 + 2 x 3 + 6 barriers of 8 bytes, the tensor-memory slot, the abort flag
constexpr int THREADS = 320;                  // warp 0: TMA, warp 1: MMA, warps 2-5 / 6-9: sigmoids of even / odd key tiles
constexpr int O_COL = 2 * BN;                  // two buffers of S (2 x BN columns; P over the first half of each), then O (D)
constexpr int TMEM_COLS = O_COL + D <= 256 ? 256 : 512;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
sigattn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                           bf16* __restrict__ out, int out_stride, const bf16* __restrict__ qf,
                           const float* __restrict__ bias, const bf16* __restrict__ gate, int gate_stride,
                           const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                           const int* __restrict__ seq_kv_len, const int* __restrict__ seq_slot,
                           const int* __restrict__ block_table, int table_stride, int Hq, int Hkv, int page_size,
                           int num_pages, int window, int k_stages, int v_stages, int skip_single, int* status) {
    extern __shared__ unsigned char smem_raw[];
    tw_grid_wait();
    // x counts (row tile, key/value head) with the head fastest and the last row tile first: the longest blocks
    // of all heads start first and the short ones fill the gaps
    const int s = blockIdx.y, kvh = (int)blockIdx.x % Hkv, xt = (int)blockIdx.x / Hkv;
    const int q_len = seq_q_len[s];
    if (q_len <= 0 || (skip_single && q_len == 1)) return;
    const int Gs = Hq / Hkv;                                         // query heads per key/value head
    const int rows_total = q_len * Gs;
    const int mtiles = (rows_total + BM - 1) / BM;
    if (xt >= mtiles) return;
    const int row0 = (mtiles - 1 - xt) * BM;
    const int kv_len = seq_kv_len[s];
    const int pos0 = kv_len - q_len;                                 // position of the first token of this portion
    const int n0 = seq_q_start[s];
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;
    const int row_end = min(rows_total, row0 + BM);
    const int pos_first = pos0 + row0 / Gs, pos_last = pos0 + (row_end - 1) / Gs;
    const int j_begin = (window > 0 && pos_first - window + 1 > 0) ? (pos_first - window + 1) / BN : 0;
    const int ntiles = pos_last / BN + 1 - j_begin;
    const int tail_rows = max(0, (j_begin + ntiles) * BN - kv_len);  // rows of the last tile that hold no key
    const int KW = Hkv * D;                                          // values of a folded query
    const int q_blocks = Hkv * KB;                                   // its 64-column blocks

    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = tiles;                                      // [q_blocks][128 rows][128 B]
    unsigned char* k_s = q_s + (size_t)q_blocks * BLK;               // [k_stages][KB][128 keys][128 B]
    unsigned char* v_s = k_s + (size_t)k_stages * CHUNK_BYTES;       // [v_stages][KB][128 keys][128 B]
    uint64_t* k_full = reinterpret_cast<uint64_t*>(v_s + (size_t)v_stages * CHUNK_BYTES);
    uint64_t* k_empty = k_full + MAX_K_STAGES;
    uint64_t* v_full = k_empty + MAX_K_STAGES;
    uint64_t* v_empty = v_full + MAX_V_STAGES;
    uint64_t* s_full = v_empty + MAX_V_STAGES;                       // S of the buffer is complete
    uint64_t* p_full = s_full + 2;                                   // P of the buffer is written
    uint64_t* o_done = p_full + 2;                                   // every product of the block has retired
    uint64_t* v_fixed = o_done + 1;                                  // value rows past the last key are zeroed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_fixed + 1);
    volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < MAX_K_STAGES; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
        for (int i = 0; i < MAX_V_STAGES; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
        for (int x = 0; x < 2; ++x) { mbar_init(&s_full[x], 1); mbar_init(&p_full[x], BM / 32); }
        mbar_init(o_done, 1);
        mbar_init(v_fixed, 1);
        *aborted = 0;
        mbar_fence_init();
    }
    // Where the boxes of key tile i lie: one TMA box per page and 64 columns of d, lane b owns box b.  The page and
    // the place inside it are the same for every key/value head and for keys and values, so they are looked up once
    // per tile (and one tile ahead: the producer's path from a free stage to the copy has no global load in it).
    const int box_rows = min(page_size, BN);
    const int boxes = BN / box_rows;
    auto look_up = [&](int i) -> int {
        int base = -1;
        if (lane < boxes && i < ntiles) {
            const int key0 = (j_begin + i) * BN + lane * box_rows;
            if (key0 < kv_len) {
                const int blk = key0 / page_size;
                const int page = blk < table_stride ? table[blk] : -1;
                if (page < 0 || page >= num_pages) atomicOr(status, TW_ERR_PAGE);
                else base = page * Hkv * page_size + (key0 - blk * page_size);
            }
        }
        return base;
    };
    // One chunk (BN keys of key/value head `head`) of the tile whose boxes start at `base`.  `use` counts the uses of
    // the ring so far.  False if a wait ran out.
    auto issue_chunk = [&](unsigned char* ring, uint64_t* full, uint64_t* empty, int stages, int use,
                           const CUtensorMap* map, int base, int head) -> bool {
        const int st = use % stages;
        const uint32_t parity = (use / stages) & 1;
        const int row_coord = base >= 0 ? base + head * page_size : -1;
        const uint32_t bytes = (uint32_t)__popc(__ballot_sync(0xffffffffu, row_coord >= 0)) * KB * box_rows * 128;
        int ok = 1;
        if (lane == 0) {
            ok = (!*aborted && mbar_wait(&empty[st], parity ^ 1, status)) ? 1 : 0;
            if (ok) mbar_expect_tx(&full[st], bytes); else *aborted = 1;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return false;
        if (row_coord >= 0) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
                tma_load_2d(ring + (size_t)st * CHUNK_BYTES + kb * KBLK + lane * box_rows * 128, map, &full[st], kb * 64, row_coord);
        }
        return true;
    };
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    // the key chunks of the first tile need nothing of what follows: the producer warp asks for as many as the ring
    // holds now, and the other warps bring the query rows in meanwhile
    int k_issued = 0, v_issued = 0;
    int base_cur = -1, base_next = -1;          // boxes of tile i and of tile i + 1 (producer warp only)
    if (warp == 0) {
        __syncwarp();
        base_cur = look_up(0);
        base_next = look_up(1);
        while (k_issued < Hkv && k_issued < k_stages &&
               issue_chunk(k_s, k_full, k_empty, k_stages, k_issued, &map_k, base_cur, k_issued)) ++k_issued;
    }
    // the block's folded query rows into shared memory, in the swizzled K-major layout (rows beyond the portion are
    // zero); eight 16-byte loads of a thread are under way before the first store
    {
        const int pieces = KW / 8;
        const int items = BM * pieces;
        constexpr int Q_THREADS = THREADS - 32;                          // every warp but the producer
        if (warp != 0) {
            for (int base = (int)threadIdx.x - 32; base < items; base += 8 * Q_THREADS) {
                uint4 vals[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = base + j * Q_THREADS;
                    vals[j] = make_uint4(0u, 0u, 0u, 0u);
                    if (i < items) {
                        const int rr = i / pieces, c = i - rr * pieces;
                        const int r = row0 + rr;
                        if (r < rows_total) {
                            const int t = r / Gs;
                            vals[j] = *reinterpret_cast<const uint4*>(
                                qf + ((size_t)(n0 + t) * Hq + kvh * Gs + (r - t * Gs)) * KW + c * 8);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int i = base + j * Q_THREADS;
                    if (i < items) {
                        const int rr = i / pieces, c = i - rr * pieces;
                        *reinterpret_cast<uint4*>(q_s + (size_t)(c >> 3) * BLK + rr * 128 + (((c & 7) ^ (rr & 7)) << 4)) = vals[j];
                    }
                }
            }
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- producer, in the order the tensor cores use things: K of tile 0; then K of tile i + 1 and V of tile i
        bool ok = !*aborted;
        while (ok && k_issued < Hkv) {
            ok = issue_chunk(k_s, k_full, k_empty, k_stages, k_issued, &map_k, base_cur, k_issued);
            if (ok) ++k_issued;
        }
        for (int i = 0; ok && i < ntiles; ++i) {
            const int base_after = look_up(i + 2);       // asked for now, used one round later
            for (int c = 0; ok && i + 1 < ntiles && c < Hkv; ++c) {
                ok = issue_chunk(k_s, k_full, k_empty, k_stages, k_issued, &map_k, base_next, c);
                if (ok) ++k_issued;
            }
            if (ok) {
                ok = issue_chunk(v_s, v_full, v_empty, v_stages, v_issued, &map_v, base_cur, kvh);
                if (ok) ++v_issued;
            }
            base_cur = base_next;
            base_next = base_after;
        }
        if (ok && tail_rows && v_issued == ntiles) {
            // The last tile reaches past the request's last key.  What its value rows hold there must not reach a
            // product, since 0 x NaN is NaN: zero them once the copies have landed, then tell the MMA thread.
            const int last = ntiles - 1;
            if (mbar_wait(&v_full[last % v_stages], (last / v_stages) & 1, status)) {
                unsigned char* vt = v_s + (size_t)(last % v_stages) * CHUNK_BYTES;
                for (int idx = lane; idx < tail_rows * KB * 8; idx += 32) {
                    const int r = BN - tail_rows + idx / (KB * 8), rest = idx % (KB * 8);
                    *reinterpret_cast<uint4*>(vt + (rest >> 3) * KBLK + r * 128 + ((rest & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(v_fixed);
            } else {
                *aborted = 1;
            }
        }
        if (*aborted && lane == 0) {
            // wait (bounded) for the copies already in flight, so that none lands after the block has gone
            for (int u = max(0, k_issued - k_stages); u < k_issued; ++u) mbar_wait(&k_full[u % k_stages], (u / k_stages) & 1, status);
            for (int u = max(0, v_issued - v_stages); u < v_issued; ++u) mbar_wait(&v_full[u % v_stages], (u / v_stages) & 1, status);
        }
    } else if (warp == 1) {
        // ---- tensor cores: lane 0 issues every MMA of the block
        if (lane == 0 && ntiles > 0) {
            const uint32_t idesc_s = instr_desc(BN), idesc_o = instr_desc(D, true);
            const uint64_t q_desc = smem_desc(q_s, 0), k_desc = smem_desc(k_s, 0), v_desc = smem_desc_mn_major(v_s, KBLK);
            int k_used = 0;
            bool ok = true;
            // S of key tile i into buffer i & 1: G chunks of the folded query against the keys of G key/value heads
            auto issue_s = [&](int i) {
                const int x = i & 1;
                for (int c = 0; ok && c < Hkv; ++c, ++k_used) {
                    const int st = k_used % k_stages;
                    ok = mbar_wait(&k_full[st], (k_used / k_stages) & 1, status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t kd = k_desc + (uint64_t)(st * (CHUNK_BYTES >> 4));
                    const uint64_t qd = q_desc + (uint64_t)(c * KB * (BLK >> 4));
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_bf16(tmem_base + x * BN, qd + (uint64_t)(kb * (BLK >> 4) + k * 2), kd + (uint64_t)(kb * (KBLK >> 4) + k * 2),
                                      idesc_s, (c > 0 || kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&k_empty[st]);
                }
                if (ok) umma_commit(&s_full[x]);
            };
            issue_s(0);
            for (int i = 0; ok && i < ntiles; ++i) {
                // S of the next tile goes to the other buffer: its P was consumed by the product issued one round ago
                if (i + 1 < ntiles) issue_s(i + 1);
                if (!ok) break;
                const int x = i & 1, vst = i % v_stages;
                ok = mbar_wait(&v_full[vst], (i / v_stages) & 1, status);
                if (ok && i == ntiles - 1 && tail_rows) ok = mbar_wait(v_fixed, 0, status);
                if (ok) ok = mbar_wait(&p_full[x], (i >> 1) & 1, status);
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = v_desc + (uint64_t)(vst * (CHUNK_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < BN / 16; ++k)
                    umma_bf16_ts(tmem_base + O_COL, tmem_base + x * BN + k * 8, vd + (uint64_t)(k * (2048 >> 4)),
                                 idesc_o, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&v_empty[vst]);
                if (i == ntiles - 1) umma_commit(o_done);
            }
            if (!ok) *aborted = 1;
        }
        __syncwarp();
    } else {
        // ---- sigmoids: thread = row rt of the block = TMEM lane rt; group x takes the key tiles i with i & 1 == x
        const int x = (warp - 2) / 4;
        const int quarter = warp & 3;                        // the TMEM lanes this warp may touch
        const int rt = quarter * 32 + lane;
        const int r = row0 + rt;
        const bool valid = r < rows_total;
        const int t = valid ? r / Gs : (rows_total - 1) / Gs;
        const int head = kvh * Gs + (valid ? r - t * Gs : 0);
        const int pos = pos0 + t;
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_addr = lane_addr + x * BN, o_addr = lane_addr + O_COL;
        constexpr float LOG2E = 1.4426950408889634f;
        const float nb = -(bias ? bias[head] : 0.f) * LOG2E;
        bool ok = true;
        for (int i = x; i < ntiles; i += 2) {
            const int kbase = (j_begin + i) * BN;
            ok = !*aborted && mbar_wait(&s_full[x], (i >> 1) & 1, status);
            if (!ok) break;
            tc_fence_after();
            uint32_t v[BN];
#pragma unroll
            for (int c = 0; c < BN; c += 32) tmem_ld32_nowait(s_addr + c, v + c);
            tmem_wait_ld();
            const bool all_visible = valid && kbase + BN - 1 <= pos && kbase >= lo;
            const bool uniform = __all_sync(0xffffffffu, all_visible);
            // p = 1 / (1 + 2^(-(s + b) log2 e)), two at a time into one 32-bit column
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                float p0 = rcp(1.0f + ex2(fmaf(__uint_as_float(v[c]), -LOG2E, nb)));
                float p1 = rcp(1.0f + ex2(fmaf(__uint_as_float(v[c + 1]), -LOG2E, nb)));
                if (!uniform) {
                    const int key = kbase + c;
                    if (!valid || key > pos || key < lo) p0 = 0.f;
                    if (!valid || key + 1 > pos || key + 1 < lo) p1 = 0.f;
                }
                v[c >> 1] = pack_bf16(p0, p1);
            }
            // P over the first half of S's columns: the whole row of S is in registers by now
#pragma unroll
            for (int c = 0; c < BN / 2; c += 32) tmem_st32_nowait(s_addr + c, v + c);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[x]);      // one arrival per warp
        }
        if (x == 0) {
            // the first group writes the block's rows: O * sigmoid(gate)
            if (ok && ntiles > 0) ok = mbar_wait(o_done, 0, status);
            if (!ok) {
                *aborted = 1;
            } else if (ntiles > 0) {
                tc_fence_after();
                bf16* orow = out + (size_t)(n0 + t) * out_stride + (size_t)head * D;
                const bf16* grow = gate ? gate + (size_t)(n0 + t) * gate_stride + (size_t)head * D : nullptr;
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t o[32];
                    tmem_ld32_nowait(o_addr + c, o);
                    tmem_wait_ld();
                    if (valid) {
#pragma unroll
                        for (int k = 0; k < 32; k += 8) {
                            float f[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[k + e]);
                            if (grow) {
                                const uint4 graw = *reinterpret_cast<const uint4*>(grow + c + k);
                                const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 gv = __bfloat1622float2(g2[e]);
                                    f[2 * e] *= rcp(1.0f + ex2(-gv.x * LOG2E));
                                    f[2 * e + 1] *= rcp(1.0f + ex2(-gv.y * LOG2E));
                                }
                            }
                            uint4 w;
                            w.x = pack_bf16(f[0], f[1]);
                            w.y = pack_bf16(f[2], f[3]);
                            w.z = pack_bf16(f[4], f[5]);
                            w.w = pack_bf16(f[6], f[7]);
                            *reinterpret_cast<uint4*>(orow + c + k) = w;
                        }
                    }
                }
            }
        } else if (!ok) {
            *aborted = 1;
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Ring depths for G key/value heads: what is left of 227 KB beside the folded queries, in chunks of one key tile; one
// to three go to the values, up to twelve to the keys.  False if fewer than three chunks fit.
bool ring_depths(int G, int* k_stages, int* v_stages, size_t* smem) {
    const long long fixed = 1024 + BARRIER_BYTES + (long long)G * KB * BLK;
    const long long n = (227ll * 1024 - fixed) / CHUNK_BYTES;
    if (n < 3) return false;
    *v_stages = n >= 9 ? 3 : (n >= 5 ? 2 : 1);
    *k_stages = (int)(n - *v_stages < MAX_K_STAGES ? n - *v_stages : MAX_K_STAGES);
    *smem = (size_t)(fixed + (long long)(*k_stages + *v_stages) * CHUNK_BYTES);
    return true;
}

}  // namespace

TW_EXPORT int tw_sigattn_tc5_head_dim() { return D; }

// Whether the kernel takes this page size and number of key/value heads: a key tile is a whole number of pages, or
// a page a whole number of key tiles, a tile has at most 32 boxes, and the folded queries leave room for the rings.
TW_EXPORT int tw_sigattn_prefill_tc5_supported(int page_size, int G) {
    int ks, vs;
    size_t smem;
    if (page_size < 4 || G <= 0) return 0;
    if (!(BN % page_size == 0 || page_size % BN == 0)) return 0;
    return ring_depths(G, &ks, &vs, &smem) ? 1 : 0;
}

// Sigmoid attention for the requests of the batch that bring several tokens (with skip_single, requests with one
// token are left to the kernel that cuts their keys into slices).  qf [tokens, Hq, Hkv * D] and out
// [tokens, Hq * D] are bf16 with 16-byte aligned rows; the cache is [pages, Hkv, page_size, D] bf16.
TW_EXPORT int tw_sigattn_prefill_tc5(void* out, int out_stride, const void* qf, const float* bias, const void* gate,
                                     int gate_stride, const int* seq_q_start, const int* seq_q_len,
                                     const int* seq_kv_len, const int* seq_slot, const int* block_table,
                                     int table_stride, const void* k_cache, const void* v_cache, int n_seqs,
                                     int max_q_len, int Hq, int Hkv, int page_size, int num_pages, int window,
                                     int skip_single, int* status, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv || !tw_sigattn_prefill_tc5_supported(page_size, Hkv)) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(qf) & 15) || (out_stride & 7) ||
        (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15) ||
        (gate && ((reinterpret_cast<uintptr_t>(gate) & 15) || (gate_stride & 7))))
        return (int)cudaErrorMisalignedAddress;
    int k_stages, v_stages;
    size_t smem;
    ring_depths(Hkv, &k_stages, &v_stages, &smem);
    cudaError_t e = cudaFuncSetAttribute(sigattn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int box_rows = page_size < BN ? page_size : BN;
    const long long rows = (long long)num_pages * Hkv * page_size;
    if (rows >= (1ll << 31)) return (int)cudaErrorInvalidValue;
    CUtensorMap mk, mv;
    if (int err = get_map(k_cache, rows, D, box_rows, &mk)) return err;
    if (int err = get_map(v_cache, rows, D, box_rows, &mv)) return err;
    const int Gs = Hq / Hkv;
    dim3 grid(((max_q_len * Gs + BM - 1) / BM) * Hkv, n_seqs);
    return tw_launch(sigattn_prefill_tc5_kernel, grid, dim3(THREADS), smem, stream, 1, mk, mv, (bf16*)out, out_stride,
                     (const bf16*)qf, bias, (const bf16*)gate, gate_stride, seq_q_start, seq_q_len, seq_kv_len, seq_slot,
                     block_table, table_stride, Hq, Hkv, page_size, num_pages, window, k_stages, v_stages, skip_single,
                     status);
}
