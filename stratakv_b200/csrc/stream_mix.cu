// Several copies of the residual stream (hyper-connections), one pass per sublayer boundary.
//
// streams [S][tokens][hidden] float.  For every token row and column w, with the old values x_s (read from `streams`, or
// all equal to source[w] where the streams have not been written yet):
//
//   update  (branch, mix, write given):  x_t <- sum_s mix[s * S + t] * x_s + write[t] * branch[w]     for all t at once
//   reading (read, gamma, normed_out):   u = sum_t read[t] * x_t;  normed_out = u / sqrt(mean_w(u^2) + eps) * gamma[w]
//   sum     (sum_out):                   sum_out[w] = sum_t x_t
//
// Everything is float; only normed_out is rounded to the compute dtype.  A block owns one token row; u is kept in
// shared memory between the pass that makes it and the pass that scales it.
#include "common.cuh"

namespace skv {

constexpr int STREAM_MIX_MAX = 8;
constexpr int STREAM_MIX_THREADS = 256;

template <typename T, int S>
__global__ void __launch_bounds__(STREAM_MIX_THREADS)
stream_mix_kernel(float* __restrict__ streams, const float* __restrict__ source, const float* __restrict__ branch,
                  const float* __restrict__ mix, const float* __restrict__ write, const float* __restrict__ read,
                  const float* __restrict__ gamma, float eps, T* __restrict__ normed_out, float* __restrict__ sum_out,
                  int n_tokens, int hidden) {
    extern __shared__ __align__(16) float stream_mix_u[];          // [hidden] when there is a reading
    __shared__ float c_mix[S * S], c_write[S], c_read[S];
    __shared__ float reduce[33];
    if (threadIdx.x < S * S) c_mix[threadIdx.x] = mix ? mix[threadIdx.x] : 0.0f;
    if (threadIdx.x < S) {
        c_write[threadIdx.x] = write ? write[threadIdx.x] : 0.0f;
        c_read[threadIdx.x] = read ? read[threadIdx.x] : 0.0f;
    }
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();
    const int t = blockIdx.x;
    const size_t plane = (size_t)n_tokens * hidden, base = (size_t)t * hidden;
    float squares = 0.0f;
    for (int w = threadIdx.x; w < hidden; w += STREAM_MIX_THREADS) {
        float x[S];
        if (source) {
            const float v = source[base + w];
#pragma unroll
            for (int s = 0; s < S; ++s) x[s] = v;
        } else {
#pragma unroll
            for (int s = 0; s < S; ++s) x[s] = streams[(size_t)s * plane + base + w];
        }
        if (branch) {
            const float y = branch[base + w];
            float fresh[S];
#pragma unroll
            for (int r = 0; r < S; ++r) {
                float acc = 0.0f;
#pragma unroll
                for (int s = 0; s < S; ++s) acc = fmaf(c_mix[s * S + r], x[s], acc);
                fresh[r] = fmaf(c_write[r], y, acc);
            }
#pragma unroll
            for (int r = 0; r < S; ++r) {
                x[r] = fresh[r];
                streams[(size_t)r * plane + base + w] = fresh[r];
            }
        }
        if (normed_out) {
            float u = 0.0f;
#pragma unroll
            for (int s = 0; s < S; ++s) u = fmaf(c_read[s], x[s], u);
            stream_mix_u[w] = u;
            squares = fmaf(u, u, squares);
        }
        if (sum_out) {
            float total = 0.0f;
#pragma unroll
            for (int s = 0; s < S; ++s) total += x[s];
            sum_out[base + w] = total;
        }
    }
    if (!normed_out) return;
    const float total = block_sum(squares, reduce);
    const float factor = 1.0f / sqrtf(total / (float)hidden + eps);
    for (int w = threadIdx.x; w < hidden; w += STREAM_MIX_THREADS)
        normed_out[base + w] = from_float<T>(stream_mix_u[w] * factor * gamma[w]);
}

template <int S>
static int launch_stream_mix(float* streams, const float* source, const float* branch, const float* mix,
                             const float* write, const float* read, const float* gamma, float eps, void* normed_out,
                             float* sum_out, int n_tokens, int hidden, cudaStream_t stream) {
    const size_t smem = normed_out ? (size_t)hidden * sizeof(float) : 0;
    auto kernel = stream_mix_kernel<skv_t, S>;
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return fail("skv_stream_mix", "the hidden size is too large");
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return fail("skv_stream_mix", "cannot reserve shared memory for a row");
    }
    return launch_pdl("skv_stream_mix", kernel, dim3(n_tokens), dim3(STREAM_MIX_THREADS), smem, stream, streams, source,
                      branch, mix, write, read, gamma, eps, (skv_t*)normed_out, sum_out, n_tokens, hidden);
}

}  // namespace skv

using namespace skv;

// Pointers that are null switch their step off (see the top of this file); `source` null: the old streams are read
// from `streams`.  mix [S * S] is indexed [from * S + to]; write, read [S]; gamma [hidden]; all float.
SKV_EXPORT int skv_stream_mix(float* streams, int n_streams, const float* source, const float* branch, const float* mix,
                              const float* write, const float* read, const float* gamma, float eps, void* normed_out,
                              float* sum_out, int n_tokens, int hidden, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!streams || hidden <= 0) return fail("skv_stream_mix", "the streams and a positive hidden size are needed");
    if (n_streams < 1 || n_streams > STREAM_MIX_MAX) return fail("skv_stream_mix", "1 to 8 streams are served");
    if ((branch != nullptr) != (mix != nullptr) || (branch != nullptr) != (write != nullptr))
        return fail("skv_stream_mix", "an update needs the sublayer's result, the mixing matrix and the write weights");
    if ((normed_out != nullptr) != (read != nullptr) || (normed_out != nullptr) != (gamma != nullptr))
        return fail("skv_stream_mix", "a reading needs the read weights, the norm's weight and a place for the result");
#define SKV_STREAM_MIX_CASE(S) \
    case S: return launch_stream_mix<S>(streams, source, branch, mix, write, read, gamma, eps, normed_out, sum_out, \
                                        n_tokens, hidden, stream);
    switch (n_streams) {
        SKV_STREAM_MIX_CASE(1) SKV_STREAM_MIX_CASE(2) SKV_STREAM_MIX_CASE(3) SKV_STREAM_MIX_CASE(4)
        SKV_STREAM_MIX_CASE(5) SKV_STREAM_MIX_CASE(6) SKV_STREAM_MIX_CASE(7) SKV_STREAM_MIX_CASE(8)
    }
#undef SKV_STREAM_MIX_CASE
    return fail("skv_stream_mix", "1 to 8 streams are served");
}
