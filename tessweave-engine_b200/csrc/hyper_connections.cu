// Hyper-connections: the residual stream is kept as `copies` parallel streams x_1 .. x_s per token
// ([rows, s, width], fp32).  A sub-layer reads a weighted sum of them and writes back into all of them:
//
//   read    u  = sum_s a[s] x_s                     h = u / sqrt(mean(u^2) + eps) * w       (the sub-layer's input)
//   write   x_t <- sum_s M[s, t] x_s + b[t] y       for all t at once, from the old copies
//
// One kernel does, for a token, whichever of these a step needs, in this order: start all copies from a given
// row; write a sub-layer's output y; read for the next sub-layer (with its norm); give the sum of the copies.
// So between two sub-layers the copies travel through the SM once.  Everything is fp32; h is rounded to the
// activation type once.  A block per token, the copies of a channel in registers.
#include "common.cuh"

#define TW_HC_MAX 16      // the most copies; kernels are compiled for up to 4, 8 and 16

template <typename T, int MAXC, int THREADS>
__global__ void __launch_bounds__(THREADS)
hyper_step_kernel(float* __restrict__ streams, const float* __restrict__ init, const T* __restrict__ y,
                  const float* __restrict__ mix, const float* __restrict__ outc, const float* __restrict__ inc,
                  const float* __restrict__ norm_w, float eps, T* __restrict__ h_out, float* __restrict__ sum_out,
                  int width, int copies) {
    extern __shared__ float su[];          // [width] the read sum, kept for the norm; then 33 floats of scratch
    __shared__ float s_mix[MAXC * MAXC], s_out[MAXC], s_in[MAXC];
    tw_grid_wait();
    tw_grid_launch_dependents();
    const int row = blockIdx.x;
    if (threadIdx.x < copies * copies && mix) s_mix[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < copies) {
        if (outc) s_out[threadIdx.x] = outc[threadIdx.x];
        if (inc) s_in[threadIdx.x] = inc[threadIdx.x];
    }
    __syncthreads();
    float* x = streams + (size_t)row * copies * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v[MAXC];
        if (init) {
            const float e = init[(size_t)row * width + c];
#pragma unroll
            for (int s = 0; s < MAXC; ++s) v[s] = e;
        } else {
#pragma unroll
            for (int s = 0; s < MAXC; ++s) v[s] = s < copies ? x[(size_t)s * width + c] : 0.f;
        }
        if (y) {
            const float yc = tw_to_float(y[(size_t)row * width + c]);
            float nv[MAXC];
#pragma unroll
            for (int t = 0; t < MAXC; ++t) {
                float acc = 0.f;
                if (t < copies) {
#pragma unroll
                    for (int s = 0; s < MAXC; ++s)
                        if (s < copies) acc += s_mix[s * copies + t] * v[s];
                    acc += s_out[t] * yc;
                }
                nv[t] = acc;
            }
#pragma unroll
            for (int t = 0; t < MAXC; ++t) v[t] = nv[t];
        }
        if (init || y) {
#pragma unroll
            for (int s = 0; s < MAXC; ++s)
                if (s < copies) x[(size_t)s * width + c] = v[s];
        }
        if (inc) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < MAXC; ++s)
                if (s < copies) u += s_in[s] * v[s];
            su[c] = u;
            ss += u * u;
        }
        if (sum_out) {
            float t = 0.f;
#pragma unroll
            for (int s = 0; s < MAXC; ++s)
                if (s < copies) t += v[s];
            sum_out[(size_t)row * width + c] = t;
        }
    }
    if (!inc) return;
    ss = tw_block_sum(ss, su + width);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        h_out[(size_t)row * width + c] = tw_from_float<T>(su[c] * inv * norm_w[c]);
}

TW_EXPORT int tw_hyper_step(float* streams, const float* init, const void* y, const float* mix, const float* outc,
                            const float* inc, const float* norm_w, float eps, void* h_out, float* sum_out, int rows,
                            int width, int copies, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (copies <= 0 || copies > TW_HC_MAX || width <= 0 || (y && (!mix || !outc)) || (inc && (!norm_w || !h_out)))
        return (int)cudaErrorInvalidValue;
    const size_t smem = ((size_t)width + 33) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    // a step of few rows is a chain of round trips to memory per thread: then a row gets a thread per channel or so
    const int threads = rows <= 64 ? min(1024, max(256, ((width + 31) / 32) * 32)) : 256;
#define TW_HC_LAUNCH_T(T, MAXC, THREADS)                                                                                   \
    do {                                                                                                                   \
        if (smem > 48 * 1024)                                                                                              \
            cudaFuncSetAttribute(hyper_step_kernel<T, MAXC, THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        return tw_launch(hyper_step_kernel<T, MAXC, THREADS>, dim3(rows), dim3(threads), smem, stream, 1, streams, init,   \
                         (const T*)y, mix, outc, inc, norm_w, eps, (T*)h_out, sum_out, width, copies);                     \
    } while (0)
#define TW_HC_LAUNCH(T, MAXC)                                                                                              \
    do {                                                                                                                   \
        if (threads > 256) TW_HC_LAUNCH_T(T, MAXC, 1024);                                                                  \
        TW_HC_LAUNCH_T(T, MAXC, 256);                                                                                      \
    } while (0)
    if (dtype == TW_F32) {
        if (copies <= 4) TW_HC_LAUNCH(float, 4);
        if (copies <= 8) TW_HC_LAUNCH(float, 8);
        TW_HC_LAUNCH(float, 16);
    }
    if (copies <= 4) TW_HC_LAUNCH(__nv_bfloat16, 4);
    if (copies <= 8) TW_HC_LAUNCH(__nv_bfloat16, 8);
    TW_HC_LAUNCH(__nv_bfloat16, 16);
#undef TW_HC_LAUNCH
#undef TW_HC_LAUNCH_T
}
