// A projection with a matrix of its own for every head (or every equal part of the channels):
//
//   out[t, h, o] = sum_i w[h, o, i] * x[t, h, i]          w [heads, out_dim, in_dim] in the compute dtype
//
// x rows are x_stride apart and out rows out_stride apart, head h starting at h * in_dim and h * out_dim; either may
// be float or the compute dtype.  Sums are float (FMA; no tensor cores, so the float32 build is true 32-bit and a
// float input, a gate of a recurrence for instance, is never rounded).  Used for block-diagonal gates and for the
// two per-head products that fold a latent's up-projections into queries and outputs.
#include "common.cuh"

namespace skv {

constexpr int HW_TOKENS = 32, HW_OUTS = 64, HW_K = 32;

template <typename TIn, typename TOut, typename TW>
__global__ void __launch_bounds__(256)
headwise_linear_kernel(const TIn* __restrict__ x, int x_stride, const TW* __restrict__ w, TOut* __restrict__ out,
                       int out_stride, int n_tokens, int in_dim, int out_dim, int zero_pad, int out_head_stride) {
    __shared__ float xs[HW_TOKENS][HW_K + 1];
    __shared__ float ws[HW_OUTS][HW_K + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.z, t0 = blockIdx.y * HW_TOKENS, o0 = blockIdx.x * HW_OUTS;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // outputs tx, tx + 16, tx + 32, tx + 48; tokens ty, ty + 16
    const TIn* x_head = x + (size_t)head * in_dim;
    const TW* w_head = w + (size_t)head * out_dim * in_dim;
    float acc[2][4] = {};
    for (int k0 = 0; k0 < in_dim; k0 += HW_K) {
        for (int idx = threadIdx.x; idx < HW_TOKENS * HW_K; idx += 256) {
            const int row = idx / HW_K, k = idx % HW_K;
            const int t = t0 + row;
            xs[row][k] = t < n_tokens && k0 + k < in_dim ? to_float(x_head[(size_t)t * x_stride + k0 + k]) : 0.0f;
        }
        for (int idx = threadIdx.x; idx < HW_OUTS * HW_K; idx += 256) {
            const int row = idx / HW_K, k = idx % HW_K;
            const int o = o0 + row;
            ws[row][k] = o < out_dim && k0 + k < in_dim ? to_float(w_head[(size_t)o * in_dim + k0 + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HW_K; ++k) {
            const float a0 = xs[ty][k], a1 = xs[ty + 16][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = ws[tx + 16 * j][k];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int t = t0 + ty + 16 * i;
        if (t >= n_tokens) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + tx + 16 * j;
            if (o < out_dim) out[(size_t)t * out_stride + (size_t)head * out_head_stride + o] = from_float<TOut>(acc[i][j]);
        }
    }
    // columns that pad a row for the projection after it are zero
    if (zero_pad && head == (int)gridDim.z - 1 && blockIdx.x == 0) {
        const int first = (int)gridDim.z * out_dim, pad = out_stride - first;
        for (int idx = threadIdx.x; idx < HW_TOKENS * pad; idx += 256) {
            const int t = t0 + idx / pad;
            if (t < n_tokens) out[(size_t)t * out_stride + first + idx % pad] = from_float<TOut>(0.0f);
        }
    }
}

template <typename TIn, typename TOut>
static int launch_headwise(const void* x, int x_stride, const void* w, void* out, int out_stride, int n_tokens,
                           int heads, int in_dim, int out_dim, int zero_pad, int out_head_stride, cudaStream_t stream) {
    const dim3 grid((out_dim + HW_OUTS - 1) / HW_OUTS, (n_tokens + HW_TOKENS - 1) / HW_TOKENS, heads);
    return launch_pdl("skv_headwise_linear", headwise_linear_kernel<TIn, TOut, skv_t>, grid, dim3(256), 0, stream,
                      (const TIn*)x, x_stride, (const skv_t*)w, (TOut*)out, out_stride, n_tokens, in_dim, out_dim, zero_pad,
                      out_head_stride);
}

}  // namespace skv

using namespace skv;

// out_head_stride: head h of an out row starts at h * out_head_stride (0: out_dim, the heads side by side).
// x_is_float / out_is_float: 1 for float, 0 for the compute dtype.  zero_pad: the columns of an out row beyond its
// heads are set to zero.
SKV_EXPORT int skv_headwise_linear(const void* x, int x_is_float, int x_stride, const void* w, void* out,
                                   int out_is_float, int out_stride, int n_tokens, int heads, int in_dim, int out_dim,
                                   int zero_pad, int out_head_stride, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || in_dim <= 0 || out_dim <= 0) return fail("skv_headwise_linear", "sizes must be positive");
    if (heads > 65535 || (n_tokens + HW_TOKENS - 1) / HW_TOKENS > 65535)
        return fail("skv_headwise_linear", "too many heads or tokens for one launch");
    if (out_head_stride <= 0) out_head_stride = out_dim;
    if (x_stride < heads * in_dim || out_head_stride < out_dim || out_stride < (heads - 1) * out_head_stride + out_dim)
        return fail("skv_headwise_linear", "a row is shorter than its heads");
    if (zero_pad && out_head_stride != out_dim)
        return fail("skv_headwise_linear", "zero_pad goes with heads that lie side by side");
    if (x_is_float && out_is_float)
        return launch_headwise<float, float>(x, x_stride, w, out, out_stride, n_tokens, heads, in_dim, out_dim, zero_pad, out_head_stride, stream);
    if (x_is_float)
        return launch_headwise<float, skv_t>(x, x_stride, w, out, out_stride, n_tokens, heads, in_dim, out_dim, zero_pad, out_head_stride, stream);
    if (out_is_float)
        return launch_headwise<skv_t, float>(x, x_stride, w, out, out_stride, n_tokens, heads, in_dim, out_dim, zero_pad, out_head_stride, stream);
    return launch_headwise<skv_t, skv_t>(x, x_stride, w, out, out_stride, n_tokens, heads, in_dim, out_dim, zero_pad, out_head_stride, stream);
}
