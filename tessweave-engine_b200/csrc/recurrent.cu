// Gated linear recurrences with a state of fixed size per request.
//
// minGRU: the gates read only the current token, so a request's rows form the first-order recurrence
//   z_t = sigmoid(pz_t + bz)         u_t = px_t + bx        c_t = u_t + 1/2 (u_t >= 0), sigmoid(u_t) (u_t < 0)
//   S_t = (1 - z_t) S_{t-1} + z_t c_t                        element by element, fp32, S_{-1} = the request's state
//   out_t = T(S_t * silu(pg_t))
// with pz | px | pg the three column blocks of one projection row.  The state slot of a request is read at
// the first row of a step and written back after its last, so a request may be cut into steps anywhere.
// Everything behind the projection is fp32.
#include "common.cuh"

#define TW_SCAN_THREADS 128

__device__ __forceinline__ float tw_sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }
// the segmented kernel's gates: accurate in float32 runs; in bfloat16 runs, whose pre-activations carry 8 bits,
// the hardware's exponential and reciprocal (fp32 all the same, a few units in the last place)
template <typename T> __device__ __forceinline__ float tw_gate_sigmoid(float x);
template <> __device__ __forceinline__ float tw_gate_sigmoid<float>(float x) { return 1.0f / (1.0f + expf(-x)); }
template <> __device__ __forceinline__ float tw_gate_sigmoid<__nv_bfloat16>(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// Short portions and single tokens: one thread per (request, channel) walks the request's rows of this step in order.
template <typename T>
__global__ void __launch_bounds__(TW_SCAN_THREADS)
mingru_scan_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ proj, int proj_stride,
                   const float* __restrict__ bias_z, const float* __restrict__ bias_x, float* __restrict__ state,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                   const int* __restrict__ seq_q_len, int width, int write_state) {
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int s = blockIdx.y;
    const int ch = blockIdx.x * TW_SCAN_THREADS + threadIdx.x;
    const int len = seq_q_len[s];
    if (ch >= width || len <= 0) return;
    const int start = seq_q_start[s];
    float* slot = state + (size_t)seq_slot[s] * width;
    float S = slot[ch];
    const float bz = bias_z ? bias_z[ch] : 0.f, bx = bias_x ? bias_x[ch] : 0.f;
    for (int t = 0; t < len; ++t) {
        const T* row = proj + (size_t)(start + t) * proj_stride;
        const float z = tw_sigmoidf(tw_to_float(row[ch]) + bz);
        const float u = tw_to_float(row[width + ch]) + bx;
        const float g = tw_to_float(row[2 * width + ch]);
        const float c = u >= 0.f ? u + 0.5f : tw_sigmoidf(u);
        S = (1.0f - z) * S + z * c;
        out[(size_t)(start + t) * out_stride + ch] = tw_from_float<T>(S * (g * tw_sigmoidf(g)));
    }
    if (write_state) slot[ch] = S;
}

// Long portions: a block of 32 warps takes 32 channels of one request; warp w walks the w-th segment of the
// request's rows from a zero state and keeps only (A, B) with S_end = A * S_in + B; the segments are chained
// in shared memory; then every warp walks its segment again from its true S_in and writes the rows.  The
// second pass finds its operands in L2.  Sums are formed in the order of the rows inside a segment and in the
// order of the segments between them, whatever the hardware does.
#define TW_SCAN_SEGMENTS 32

template <typename T>
__global__ void __launch_bounds__(32 * TW_SCAN_SEGMENTS)
mingru_scan_segments_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ proj, int proj_stride,
                            const float* __restrict__ bias_z, const float* __restrict__ bias_x, float* __restrict__ state,
                            const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                            const int* __restrict__ seq_q_len, int width, int write_state) {
    __shared__ float sA[TW_SCAN_SEGMENTS][33], sB[TW_SCAN_SEGMENTS][33];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int s = blockIdx.y;
    const int lane = threadIdx.x & 31, seg = threadIdx.x >> 5;
    const int ch = blockIdx.x * 32 + lane;
    const int len = seq_q_len[s];
    if (len <= 0) return;
    const bool live = ch < width;
    const int start = seq_q_start[s];
    const int per = (len + TW_SCAN_SEGMENTS - 1) / TW_SCAN_SEGMENTS;
    const int t0 = min(len, seg * per), t1 = min(len, t0 + per);
    const float bz = (live && bias_z) ? bias_z[ch] : 0.f, bx = (live && bias_x) ? bias_x[ch] : 0.f;
    float A = 1.f, B = 0.f;
    if (live) {
        // the loads and gates of a row do not depend on the row before: eight rows at a time, so that their
        // round trips to memory overlap, then the eight steps of the recurrence in order
        int t = t0;
        for (; t + 8 <= t1; t += 8) {
            float zs[8], cs[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const T* row = proj + (size_t)(start + t + k) * proj_stride;
                zs[k] = tw_to_float(row[ch]);
                cs[k] = tw_to_float(row[width + ch]);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float z = tw_gate_sigmoid<T>(zs[k] + bz);
                const float u = cs[k] + bx;
                const float c = u >= 0.f ? u + 0.5f : tw_gate_sigmoid<T>(u);
                A *= 1.0f - z;
                B = (1.0f - z) * B + z * c;
            }
        }
        for (; t < t1; ++t) {
            const T* row = proj + (size_t)(start + t) * proj_stride;
            const float z = tw_gate_sigmoid<T>(tw_to_float(row[ch]) + bz);
            const float u = tw_to_float(row[width + ch]) + bx;
            const float c = u >= 0.f ? u + 0.5f : tw_gate_sigmoid<T>(u);
            A *= 1.0f - z;
            B = (1.0f - z) * B + z * c;
        }
    }
    sA[seg][lane] = A;
    sB[seg][lane] = B;
    __syncthreads();
    float* slot = state + (size_t)seq_slot[s] * width;
    if (seg == 0 && live) {
        float S = slot[ch];
        for (int k = 0; k < TW_SCAN_SEGMENTS; ++k) {
            const float a = sA[k][lane], b = sB[k][lane];
            sA[k][lane] = S;                 // what segment k starts from
            S = a * S + b;
        }
        if (write_state) slot[ch] = S;
    }
    __syncthreads();
    if (!live) return;
    float S = sA[seg][lane];
    int t = t0;
    for (; t + 8 <= t1; t += 8) {
        float zs[8], cs[8], gs[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const T* row = proj + (size_t)(start + t + k) * proj_stride;
            zs[k] = tw_to_float(row[ch]);
            cs[k] = tw_to_float(row[width + ch]);
            gs[k] = tw_to_float(row[2 * width + ch]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float z = tw_gate_sigmoid<T>(zs[k] + bz);
            const float u = cs[k] + bx;
            const float c = u >= 0.f ? u + 0.5f : tw_gate_sigmoid<T>(u);
            S = (1.0f - z) * S + z * c;
            out[(size_t)(start + t + k) * out_stride + ch] = tw_from_float<T>(S * (gs[k] * tw_gate_sigmoid<T>(gs[k])));
        }
    }
    for (; t < t1; ++t) {
        const T* row = proj + (size_t)(start + t) * proj_stride;
        const float z = tw_gate_sigmoid<T>(tw_to_float(row[ch]) + bz);
        const float u = tw_to_float(row[width + ch]) + bx;
        const float g = tw_to_float(row[2 * width + ch]);
        const float c = u >= 0.f ? u + 0.5f : tw_gate_sigmoid<T>(u);
        S = (1.0f - z) * S + z * c;
        out[(size_t)(start + t) * out_stride + ch] = tw_from_float<T>(S * (g * tw_gate_sigmoid<T>(g)));
    }
}

TW_EXPORT int tw_mingru_scan(void* out, int out_stride, const void* proj, int proj_stride, const float* bias_z,
                             const float* bias_x, float* state, const int* seq_slot, const int* seq_q_start,
                             const int* seq_q_len, int n_seqs, int max_q_len, int width, int write_state, int dtype,
                             cudaStream_t stream) {
    if (n_seqs <= 0 || width <= 0) return 0;
    if (max_q_len > 2 * TW_SCAN_SEGMENTS) {
        const dim3 grid((width + 31) / 32, n_seqs);
        if (dtype == TW_F32)
            return tw_launch(mingru_scan_segments_kernel<float>, grid, dim3(32 * TW_SCAN_SEGMENTS), 0, stream, 1, (float*)out,
                             out_stride, (const float*)proj, proj_stride, bias_z, bias_x, state, seq_slot, seq_q_start,
                             seq_q_len, width, write_state);
        return tw_launch(mingru_scan_segments_kernel<__nv_bfloat16>, grid, dim3(32 * TW_SCAN_SEGMENTS), 0, stream, 1,
                         (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)proj, proj_stride, bias_z, bias_x, state,
                         seq_slot, seq_q_start, seq_q_len, width, write_state);
    }
    const dim3 grid((width + TW_SCAN_THREADS - 1) / TW_SCAN_THREADS, n_seqs);
    if (dtype == TW_F32)
        return tw_launch(mingru_scan_kernel<float>, grid, dim3(TW_SCAN_THREADS), 0, stream, 1, (float*)out, out_stride,
                         (const float*)proj, proj_stride, bias_z, bias_x, state, seq_slot, seq_q_start, seq_q_len, width,
                         write_state);
    return tw_launch(mingru_scan_kernel<__nv_bfloat16>, grid, dim3(TW_SCAN_THREADS), 0, stream, 1, (__nv_bfloat16*)out,
                     out_stride, (const __nv_bfloat16*)proj, proj_stride, bias_z, bias_x, state, seq_slot, seq_q_start,
                     seq_q_len, width, write_state);
}
