// Sigmoid attention with mixed heads over a paged cache: preparation of queries and keys, and the
// exact-arithmetic attention kernel (fp32 scores and sums, any sizes, float32 or bfloat16 storage).
//
// The mechanism, for a token at position i of a request with H query heads, G key/value heads of size D
// (query head h reads key/value head c(h) = h / (H / G)):
//
//   q = rms(Wq x) * nq, k = rms(Wk x) * nk       each norm over the WHOLE projection (all heads at once)
//   v = Wk x                                      the values are the keys as projected: no norm, no rotation
//   q, k rotated by position on the first R dims of every head
//   s_g(i, j)  = scale * q_g(i) . k_c(g)(j)
//   s'_h(i, j) = sum_g M[h, g] s_g(i, j)          M: H x H, mixes the heads' scores
//   w_h(i, j)  = sigmoid(s'_h(i, j) + b_h)        j <= i [and j > i - window]; never normalised over j
//   o_h(i)     = sum_j w_h(i, j) v_c(h)(j)        then o * sigmoid(gate) where a gate is given
//
// The mixing is linear in the queries, so it is done once per token instead of once per (token, key):
//   s'_h(i, j) = sum_c qf_h,c(i) . k_c(j),   qf_h,c = scale * sum_{g in group c} M[h, g] q_g
// The "folded" query of head h is the row [qf_h,0 | qf_h,1 | ...] of G * D values and meets the keys of ALL
// key/value heads of a position; after that every head is an ordinary attention head whose weight is a sigmoid.
// Without M (null) the fold is scale * q_h in its own group's columns and zero elsewhere.
#include "common.cuh"

#define TW_SIG_PREP_THREADS 256

// ---------------------------------------------------------------------------------------
// Preparation, one block per token: norms over the whole projections, rotation, the raw key into the
// value pages, the normalised rotated key into the key pages, the folded query into `qf`.
//   proj row: [q heads | k heads | ...] (what follows is not touched)
//   rotation: angle = float(position) * inv_freq[i], i < rot_dims / 2; pair (2i, 2i+1) of a head when
//   `interleaved`, else (i, i + rot_dims / 2); dims from rot_dims on pass unchanged.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(TW_SIG_PREP_THREADS)
sigattn_prepare_kernel(const T* __restrict__ proj, int proj_stride, const float* __restrict__ q_norm_w,
                       const float* __restrict__ k_norm_w, float eps, const float* __restrict__ mix, float scale,
                       const float* __restrict__ inv_freq, int rot_dims, int interleaved,
                       const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                       const int* __restrict__ seq_slot, const int* __restrict__ block_table, int table_stride,
                       T* __restrict__ qf, T* __restrict__ k_cache, T* __restrict__ v_cache, int Hq, int Hkv, int D,
                       int page_size, int num_pages, int write_cache, int* status) {
    // q: Hq * D, k: Hkv * D, cos and sin: rot_dims / 2 each, the mixing matrix: Hq * Hq, then 33 floats for the reductions
    extern __shared__ __align__(16) float smem[];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    const int s = seq_of_token[n];
    if (s < 0) return;                       // padding row of a fixed-size batch
    // With few rows the heads of a token are shared out over gridDim.y blocks: each block forms the norms (it needs
    // the whole rows for them) and the rotation, folds the queries of its own heads, and block 0 writes the cache.
    const int part = blockIdx.y, parts = gridDim.y;
    const int pos = positions[n];
    const int QW = Hq * D, KW = Hkv * D;
    const int half = rot_dims >> 1;
    float* sq = smem;
    float* sk = sq + QW;
    float* s_cos = sk + KW;
    float* s_sin = s_cos + half;
    float* s_mix = s_sin + half;
    float* scratch = s_mix + (mix ? Hq * Hq : 0);
    const T* row = proj + (size_t)n * proj_stride;

    int page = -1;
    if (write_cache && part == 0) {
        const int blk = pos / page_size;
        page = blk < table_stride ? block_table[(size_t)seq_slot[s] * table_stride + blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(status, TW_ERR_PAGE);
            page = -1;
        }
    }
    const int in_page = pos % page_size;
    // the angles depend on the position and the pair only: each is evaluated once per block, not once per head
    if (inv_freq) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    if (mix) {
        for (int i = threadIdx.x; i < Hq * Hq; i += blockDim.x) s_mix[i] = mix[i];
    }
    float ssq = 0.f, ssk = 0.f;
    for (int i = threadIdx.x; i < QW; i += blockDim.x) {
        const float v = tw_to_float(row[i]);
        sq[i] = v;
        ssq += v * v;
    }
    for (int i = threadIdx.x; i < KW; i += blockDim.x) {
        const T raw = row[QW + i];
        const float v = tw_to_float(raw);
        sk[i] = v;
        ssk += v * v;
        if (page >= 0) {                     // the value is the key as projected
            const int c = i / D, d = i - c * D;
            v_cache[(((size_t)page * Hkv + c) * page_size + in_page) * D + d] = raw;
        }
    }
    ssq = tw_block_sum(ssq, scratch);
    ssk = tw_block_sum(ssk, scratch);
    const float inv_q = 1.0f / sqrtf(ssq / (float)QW + eps);
    const float inv_k = 1.0f / sqrtf(ssk / (float)KW + eps);
    for (int i = threadIdx.x; i < QW; i += blockDim.x) sq[i] = (sq[i] * inv_q) * q_norm_w[i];
    for (int i = threadIdx.x; i < KW; i += blockDim.x) sk[i] = (sk[i] * inv_k) * k_norm_w[i];
    __syncthreads();
    if (inv_freq && half > 0) {
        const int pairs = (Hq + Hkv) * half;
        for (int idx = threadIdx.x; idx < pairs; idx += blockDim.x) {
            const int head = idx / half, i = idx - head * half;
            float* base = (head < Hq ? sq + head * D : sk + (head - Hq) * D);
            const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
            const float sn = s_sin[i], cs = s_cos[i];
            const float u = base[a], v = base[b];
            base[a] = u * cs - v * sn;
            base[b] = v * cs + u * sn;
        }
        __syncthreads();
    }
    if (page >= 0) {
        for (int i = threadIdx.x; i < KW; i += blockDim.x) {
            const int c = i / D, d = i - c * D;
            k_cache[(((size_t)page * Hkv + c) * page_size + in_page) * D + d] = tw_from_float<T>(sk[i]);
        }
    }
    const int group = Hq / Hkv;
    const int h_per = (Hq + parts - 1) / parts;
    const int h_lo = part * h_per, h_hi = min(Hq, h_lo + h_per);
    T* out = qf + (size_t)n * Hq * KW;
    if (mix && (D & 3) == 0) {
        // a thread owns four neighbouring columns (c, d .. d + 3) of the folded rows and eight heads at a time: one
        // 16-byte read of q per head of the group, one broadcast read of the mixing matrix per four products
        for (int rem4 = threadIdx.x; rem4 < (KW >> 2); rem4 += blockDim.x) {
            const int rem = rem4 << 2;
            const int c = rem / D, d = rem - c * D;
            const float* q = sq + (c * group) * D + d;
            for (int hb = h_lo; hb < h_hi; hb += 8) {
                float4 acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int g = 0; g < group; ++g) {
                    const float4 qv = *reinterpret_cast<const float4*>(q + g * D);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (hb + j < h_hi) {
                            const float m = s_mix[(hb + j) * Hq + c * group + g];
                            acc[j].x += m * qv.x; acc[j].y += m * qv.y; acc[j].z += m * qv.z; acc[j].w += m * qv.w;
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (hb + j < h_hi) {
                        T* dst = out + (size_t)(hb + j) * KW + rem;
                        dst[0] = tw_from_float<T>(acc[j].x * scale);
                        dst[1] = tw_from_float<T>(acc[j].y * scale);
                        dst[2] = tw_from_float<T>(acc[j].z * scale);
                        dst[3] = tw_from_float<T>(acc[j].w * scale);
                    }
                }
            }
        }
        return;
    }
    // any head size, or no mixing: a thread owns columns (c, d) of the folded rows and walks the block's heads
    for (int rem = threadIdx.x; rem < KW; rem += blockDim.x) {
        const int c = rem / D, d = rem - c * D;
        const float* q = sq + (c * group) * D + d;
        for (int h = h_lo; h < h_hi; ++h) {
            float acc = 0.f;
            if (mix) {
                const float* m = s_mix + h * Hq + c * group;
                for (int g = 0; g < group; ++g) acc += m[g] * q[g * D];
            } else if (h / group == c) {
                acc = sq[h * D + d];
            }
            out[(size_t)h * KW + rem] = tw_from_float<T>(acc * scale);
        }
    }
}

// The same for bfloat16 rows whose head size is a multiple of 8 and whose rotation pairs neighbours (or is absent):
// eight values per access.  A thread that normalises a piece also rotates it (both values of a pair are its own),
// and a piece of k goes from registers straight to its page.
__device__ __forceinline__ void tw_unpack8(const uint4& raw, float (&x)[8]) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        x[2 * e] = f.x;
        x[2 * e + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 tw_pack8(const float (&x)[8]) {
    uint4 raw;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(x[2 * e], x[2 * e + 1]);
    return raw;
}

__global__ void __launch_bounds__(TW_SIG_PREP_THREADS)
sigattn_prepare_bf16x8_kernel(const __nv_bfloat16* __restrict__ proj, int proj_stride, const float* __restrict__ q_norm_w,
                              const float* __restrict__ k_norm_w, float eps, const float* __restrict__ mix, float scale,
                              const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
                              const int* __restrict__ seq_of_token, const int* __restrict__ seq_slot,
                              const int* __restrict__ block_table, int table_stride, __nv_bfloat16* __restrict__ qf,
                              __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int Hq, int Hkv, int D,
                              int page_size, int num_pages, int write_cache, int* status) {
    extern __shared__ __align__(16) float smem[];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int n = blockIdx.x;
    const int s = seq_of_token[n];
    if (s < 0) return;
    const int part = blockIdx.y, parts = gridDim.y;
    const int pos = positions[n];
    const int QW = Hq * D, KW = Hkv * D;
    const int half = rot_dims >> 1;
    float* sq = smem;
    float* sk = sq + QW;
    float* s_cos = sk + KW;
    float* s_sin = s_cos + half;
    float* s_mix = s_sin + half;
    float* scratch = s_mix + (mix ? Hq * Hq : 0);
    const uint4* row = reinterpret_cast<const uint4*>(proj + (size_t)n * proj_stride);
    int page = -1;
    if (write_cache && part == 0) {
        const int blk = pos / page_size;
        page = blk < table_stride ? block_table[(size_t)seq_slot[s] * table_stride + blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(status, TW_ERR_PAGE);
            page = -1;
        }
    }
    const int in_page = pos % page_size;
    if (inv_freq) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &s_sin[i], &s_cos[i]);
    }
    if (mix) {
        for (int i = threadIdx.x; i < Hq * Hq; i += blockDim.x) s_mix[i] = mix[i];
    }
    const int q8 = QW >> 3, all8 = (QW + KW) >> 3;
    float ssq = 0.f, ssk = 0.f;
    for (int i = threadIdx.x; i < all8; i += blockDim.x) {
        const uint4 raw = row[i];
        float x[8];
        tw_unpack8(raw, x);
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
        float* dst = i < q8 ? sq + 8 * i : sk + 8 * (i - q8);
        *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(x[4], x[5], x[6], x[7]);
        if (i < q8) {
            ssq += ss;
        } else {
            ssk += ss;
            if (page >= 0) {                 // the value is the key as projected
                const int col = 8 * (i - q8), c = col / D, d = col - c * D;
                *reinterpret_cast<uint4*>(v_cache + (((size_t)page * Hkv + c) * page_size + in_page) * D + d) = raw;
            }
        }
    }
    ssq = tw_block_sum(ssq, scratch);
    ssk = tw_block_sum(ssk, scratch);
    const float inv_q = 1.0f / sqrtf(ssq / (float)QW + eps);
    const float inv_k = 1.0f / sqrtf(ssk / (float)KW + eps);
    for (int i = threadIdx.x; i < all8; i += blockDim.x) {
        const bool is_q = i < q8;
        const int col = is_q ? 8 * i : 8 * (i - q8);
        float* src = (is_q ? sq : sk) + col;
        const float* wsrc = (is_q ? q_norm_w : k_norm_w) + col;
        const float inv = is_q ? inv_q : inv_k;
        if (!is_q && page < 0) continue;     // nobody reads this block's k
        const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
        const float4 wa = *reinterpret_cast<const float4*>(wsrc), wb = *reinterpret_cast<const float4*>(wsrc + 4);
        float x[8] = {(a.x * inv) * wa.x, (a.y * inv) * wa.y, (a.z * inv) * wa.z, (a.w * inv) * wa.w,
                      (b.x * inv) * wb.x, (b.y * inv) * wb.y, (b.z * inv) * wb.z, (b.w * inv) * wb.w};
        const int head = col / D, d0 = col - head * D;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int pi = (d0 >> 1) + j;
            if (pi < half) {
                const float sn = s_sin[pi], cs = s_cos[pi];
                const float u = x[2 * j], v = x[2 * j + 1];
                x[2 * j] = u * cs - v * sn;
                x[2 * j + 1] = v * cs + u * sn;
            }
        }
        if (is_q) {
            *reinterpret_cast<float4*>(src) = make_float4(x[0], x[1], x[2], x[3]);
            *reinterpret_cast<float4*>(src + 4) = make_float4(x[4], x[5], x[6], x[7]);
        } else {
            *reinterpret_cast<uint4*>(k_cache + (((size_t)page * Hkv + head) * page_size + in_page) * D + d0) = tw_pack8(x);
        }
    }
    __syncthreads();
    const int group = Hq / Hkv;
    const int h_per = (Hq + parts - 1) / parts;
    const int h_lo = part * h_per, h_hi = min(Hq, h_lo + h_per);
    __nv_bfloat16* out = qf + (size_t)n * Hq * KW;
    // a thread owns four neighbouring columns of the folded rows; where a row has fewer groups of four than the block
    // has threads, the block's heads are shared out over the threads that own the same columns, eight at a time
    const int col_groups = KW >> 2;
    const int sharers = col_groups < (int)blockDim.x ? (int)blockDim.x / col_groups : 1;
    const int share = sharers > 1 ? (int)threadIdx.x / col_groups : 0;
    for (int rem4 = sharers > 1 ? (int)threadIdx.x % col_groups : (int)threadIdx.x;
         rem4 < col_groups && share < sharers; rem4 += blockDim.x) {
        const int rem = rem4 << 2;
        const int c = rem / D, d = rem - c * D;
        const float* q = sq + (c * group) * D + d;
        for (int hb = h_lo + 8 * share; hb < h_hi; hb += 8 * sharers) {
            float4 acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (mix) {
                for (int g = 0; g < group; ++g) {
                    const float4 qv = *reinterpret_cast<const float4*>(q + g * D);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (hb + j < h_hi) {
                            const float m = s_mix[(hb + j) * Hq + c * group + g];
                            acc[j].x += m * qv.x; acc[j].y += m * qv.y; acc[j].z += m * qv.z; acc[j].w += m * qv.w;
                        }
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (hb + j < h_hi && (hb + j) / group == c) acc[j] = *reinterpret_cast<const float4*>(sq + (hb + j) * D + d);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (hb + j < h_hi) {
                    uint2 w;
                    *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(acc[j].x * scale, acc[j].y * scale);
                    *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(acc[j].z * scale, acc[j].w * scale);
                    *reinterpret_cast<uint2*>(out + (size_t)(hb + j) * KW + rem) = w;
                }
            }
        }
    }
}

TW_EXPORT int tw_sigattn_prepare(const void* proj, int proj_stride, const float* q_norm_w, const float* k_norm_w,
                                 float eps, const float* mix, float scale, const float* inv_freq, int rot_dims,
                                 int interleaved, const int* positions, const int* seq_of_token, const int* seq_slot,
                                 const int* block_table, int table_stride, void* qf, void* k_cache, void* v_cache,
                                 int n_tokens, int Hq, int Hkv, int D, int page_size, int num_pages, int write_cache,
                                 int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || Hkv <= 0 || Hq % Hkv || rot_dims < 0 || rot_dims > D || (rot_dims & 1)) return (int)cudaErrorInvalidValue;
    if (!inv_freq) rot_dims = 0;
    const size_t smem = ((size_t)(Hq + Hkv) * D + rot_dims + (mix ? (size_t)Hq * Hq : 0) + 33) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    // few rows: up to eight blocks per token, so that a decode step does not leave this to a handful of SMs
    int parts = 1;
    if (n_tokens < 148) parts = Hq < 8 ? Hq : 8;
    const dim3 grid(n_tokens, parts);
    cudaError_t e;
    if (dtype == TW_F32) {
        e = cudaFuncSetAttribute(sigattn_prepare_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        return tw_launch(sigattn_prepare_kernel<float>, grid, dim3(TW_SIG_PREP_THREADS), smem, stream, 1,
                         (const float*)proj, proj_stride, q_norm_w, k_norm_w, eps, mix, scale, inv_freq, rot_dims,
                         interleaved, positions, seq_of_token, seq_slot, block_table, table_stride, (float*)qf,
                         (float*)k_cache, (float*)v_cache, Hq, Hkv, D, page_size, num_pages, write_cache, status);
    }
    const bool aligned = !((reinterpret_cast<uintptr_t>(proj) | reinterpret_cast<uintptr_t>(qf) | reinterpret_cast<uintptr_t>(k_cache) |
                            reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(q_norm_w) |
                            reinterpret_cast<uintptr_t>(k_norm_w)) & 15);
    if ((D & 7) == 0 && (proj_stride & 7) == 0 && aligned && (interleaved || !inv_freq)) {
        e = cudaFuncSetAttribute(sigattn_prepare_bf16x8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        return tw_launch(sigattn_prepare_bf16x8_kernel, grid, dim3(TW_SIG_PREP_THREADS), smem, stream, 1,
                         (const __nv_bfloat16*)proj, proj_stride, q_norm_w, k_norm_w, eps, mix, scale, inv_freq, rot_dims,
                         positions, seq_of_token, seq_slot, block_table, table_stride, (__nv_bfloat16*)qf,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, D, page_size, num_pages, write_cache,
                         status);
    }
    e = cudaFuncSetAttribute(sigattn_prepare_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return tw_launch(sigattn_prepare_kernel<__nv_bfloat16>, grid, dim3(TW_SIG_PREP_THREADS), smem, stream, 1,
                     (const __nv_bfloat16*)proj, proj_stride, q_norm_w, k_norm_w, eps, mix, scale, inv_freq, rot_dims,
                     interleaved, positions, seq_of_token, seq_slot, block_table, table_stride, (__nv_bfloat16*)qf,
                     (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, D, page_size, num_pages, write_cache,
                     status);
}

// ---------------------------------------------------------------------------------------
// Exact attention, one block per (token, head): the folded query (G * D values, fp32 in shared memory)
// meets the keys lo..position of its request, key p in warp p % 4, so the order of the sums at a
// position depends neither on how the request was cut into steps nor on what else is in the batch.
//   w = 1 / (1 + exp(-(qf . k + bias[head])))        acc += w * v_c(head)
// gate (may be null): out *= 1 / (1 + exp(-gate[n, head * D + d])).
// ---------------------------------------------------------------------------------------
#define TW_SIG_WARPS 4
#define TW_SIG_MAXR 8       // head_dim <= 32 * 8

template <typename T>
__global__ void __launch_bounds__(32 * TW_SIG_WARPS)
sigattn_generic_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ qf, const float* __restrict__ bias,
                       const T* __restrict__ gate, int gate_stride, const int* __restrict__ positions,
                       const int* __restrict__ seq_of_token, const int* __restrict__ seq_slot,
                       const int* __restrict__ block_table, int table_stride, const T* __restrict__ k_cache,
                       const T* __restrict__ v_cache, int Hq, int Hkv, int D, int page_size, int num_pages, int window,
                       int* status) {
    extern __shared__ float smem[];          // folded query: Hkv * D; then TW_SIG_WARPS * D for the merge
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int n = blockIdx.x, head = blockIdx.y;
    const int s = seq_of_token[n];
    if (s < 0) return;
    const int pos = positions[n];
    const int KW = Hkv * D;
    const int kvh = head / (Hq / Hkv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int* table = block_table + (size_t)seq_slot[s] * table_stride;
    float* sqf = smem;
    float* merge = smem + KW;
    const T* qrow = qf + ((size_t)n * Hq + head) * KW;
    for (int i = threadIdx.x; i < KW; i += blockDim.x) sqf[i] = tw_to_float(qrow[i]);
    __syncthreads();
    const float b = bias ? bias[head] : 0.f;
    float acc[TW_SIG_MAXR];
#pragma unroll
    for (int j = 0; j < TW_SIG_MAXR; ++j) acc[j] = 0.f;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    int p = lo + ((warp - lo) % TW_SIG_WARPS + TW_SIG_WARPS) % TW_SIG_WARPS;
    for (; p <= pos; p += TW_SIG_WARPS) {
        const int blk = p / page_size;
        const int page = blk < table_stride ? table[blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0) atomicOr(status, TW_ERR_PAGE);
            continue;
        }
        const int in_page = p - blk * page_size;
        float dot = 0.f;
        for (int c = 0; c < Hkv; ++c) {
            const T* kr = k_cache + (((size_t)page * Hkv + c) * page_size + in_page) * D;
            const float* qc = sqf + c * D;
            for (int d = lane; d < D; d += 32) dot += qc[d] * tw_to_float(kr[d]);
        }
        dot = tw_warp_sum(dot);
        const float w = 1.0f / (1.0f + expf(-(dot + b)));
        const T* vr = v_cache + (((size_t)page * Hkv + kvh) * page_size + in_page) * D;
#pragma unroll
        for (int j = 0; j < TW_SIG_MAXR; ++j) {
            const int d = lane + 32 * j;
            if (d < D) acc[j] += w * tw_to_float(vr[d]);
        }
    }
    float* my = merge + warp * D;
#pragma unroll
    for (int j = 0; j < TW_SIG_MAXR; ++j) {
        const int d = lane + 32 * j;
        if (d < D) my[d] = acc[j];
    }
    __syncthreads();
    T* orow = out + (size_t)n * out_stride + head * D;
    const T* grow = gate ? gate + (size_t)n * gate_stride + head * D : nullptr;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < TW_SIG_WARPS; ++w) o += merge[w * D + d];
        if (grow) o *= 1.0f / (1.0f + expf(-tw_to_float(grow[d])));
        orow[d] = tw_from_float<T>(o);
    }
}

TW_EXPORT int tw_sigattn_generic(void* out, int out_stride, const void* qf, const float* bias, const void* gate,
                                 int gate_stride, const int* positions, const int* seq_of_token, const int* seq_slot,
                                 const int* block_table, int table_stride, const void* k_cache, const void* v_cache,
                                 int n_tokens, int Hq, int Hkv, int D, int page_size, int num_pages, int window,
                                 int dtype, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || D > 32 * TW_SIG_MAXR || Hkv <= 0 || Hq % Hkv) return (int)cudaErrorInvalidValue;
    const dim3 grid(n_tokens, Hq);
    const size_t smem = ((size_t)Hkv * D + (size_t)TW_SIG_WARPS * D) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    cudaError_t e;
    if (dtype == TW_F32) {
        e = cudaFuncSetAttribute(sigattn_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        return tw_launch(sigattn_generic_kernel<float>, grid, dim3(32 * TW_SIG_WARPS), smem, stream, 1, (float*)out,
                         out_stride, (const float*)qf, bias, (const float*)gate, gate_stride, positions, seq_of_token,
                         seq_slot, block_table, table_stride, (const float*)k_cache, (const float*)v_cache, Hq, Hkv, D,
                         page_size, num_pages, window, status);
    }
    e = cudaFuncSetAttribute(sigattn_generic_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return tw_launch(sigattn_generic_kernel<__nv_bfloat16>, grid, dim3(32 * TW_SIG_WARPS), smem, stream, 1,
                     (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)qf, bias, (const __nv_bfloat16*)gate,
                     gate_stride, positions, seq_of_token, seq_slot, block_table, table_stride,
                     (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, Hq, Hkv, D, page_size, num_pages,
                     window, status);
}
