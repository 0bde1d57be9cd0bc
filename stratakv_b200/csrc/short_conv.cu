// Steps between a fused projection and attention that the head-wise finish (attention_general.cu) does not have:
//
//   projection_norm:    an RMS norm with a weight over a whole segment of a projection's float rows (all query heads
//                       together, all key heads together), the segment's bias added first, in place;
//   short_conv_rotary:  a short causal convolution over time on every channel of the queries and keys,
//                           y_p = sum_j w[c][j] * u_(p - taps + 1 + j)       (u: the biased projection; zero before p = 0)
//                       then rotary positions on the first `rotated` numbers of every head (pairs (2i, 2i+1) or
//                       (i, i + rotated/2)), queries to q_out, rotated keys into the paged key cache and, where the
//                       values are the keys, the convolved keys before rotation into the value cache;
//   short_conv_remember: the biased projections of a sequence's last taps - 1 positions into its state.
//
// Per sequence the cache keeps float state, one row per slot, starting `state_offset` floats into the row:
//   [taps][channels]  the biased projection of the last positions, at row (position mod taps).  short_conv_rotary reads
//                     the rows of positions before the step; short_conv_remember, a later kernel of the same step,
//                     writes the rows of the step's own last positions: a one-token step writes the one row that none of
//                     its own taps reads, so it may run twice.
#include "common.cuh"

namespace skv {

struct NormSegment {
    int offset, width;
    const float* bias;         // [width] or null
    const float* weight;       // [width]
};

// grid (tokens, segments)
__global__ void __launch_bounds__(256)
projection_norm_kernel(float* __restrict__ rows, int row_stride, float eps, const NormSegment first,
                       const NormSegment second) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const NormSegment seg = blockIdx.y == 0 ? first : second;
    float* x = rows + (size_t)blockIdx.x * row_stride + seg.offset;
    float squares = 0.0f;
    for (int c = threadIdx.x; c < seg.width; c += blockDim.x) {
        const float v = x[c] + (seg.bias ? seg.bias[c] : 0.0f);
        squares = fmaf(v, v, squares);
    }
    const float factor = 1.0f / sqrtf(block_sum(squares, scratch) / (float)seg.width + eps);
    for (int c = threadIdx.x; c < seg.width; c += blockDim.x)
        x[c] = (x[c] + (seg.bias ? seg.bias[c] : 0.0f)) * factor * seg.weight[c];
}

struct ConvBatch {
    const int* positions;      // [tokens]
    const int* token_seq;      // [tokens]
    const int* cu_q;           // [seqs + 1]
    const int* slot_ids;       // [seqs]
    float* state;              // [slots][state_stride] floats
    long long state_stride;
    long long state_offset;
};

// The convolved value of channel c at token t (position p of sequence s, whose first token of the step is `first`).
__device__ __forceinline__ float convolved(const float* __restrict__ rows, int row_stride, const float* __restrict__ bias,
                                           const float* __restrict__ conv_w, const float* __restrict__ ring, int channels,
                                           int taps, int t, int p, int first, int c) {
    const float b = bias ? bias[c] : 0.0f;
    if (taps <= 1) return (rows[(size_t)t * row_stride + c] + b) * (taps == 1 ? conv_w[c] : 1.0f);
    float sum = 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;
        if (p - back < 0) continue;
        const float u = t - back >= first ? rows[(size_t)(t - back) * row_stride + c] + b
                                          : ring[(size_t)((p - back) % taps) * channels + c];
        sum = fmaf(conv_w[(size_t)c * taps + j], u, sum);
    }
    return sum;
}

// A warp per (token, head): the token's query heads, then its key heads.  rows [tokens, row_stride] float holds
// [queries | keys]; conv_w [channels, taps] and bias [channels] cover the same columns (taps 0: no convolution).
template <typename T>
__global__ void __launch_bounds__(256)
short_conv_rotary_kernel(const float* __restrict__ rows, int row_stride, const float* __restrict__ bias,
                         const float* __restrict__ conv_w, int taps, const float2* __restrict__ cos_sin, int rotated,
                         int interleaved, const int* __restrict__ block_table, int table_width, T* __restrict__ q_out,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, int n_tokens, int num_heads, int num_kv_heads,
                         int dim, int block_size, int write_kv, const ConvBatch batch) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int per_token = num_heads + num_kv_heads;
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * per_token) return;
    const int t = (int)(item / per_token), which = (int)(item - (long long)t * per_token);
    const bool is_query = which < num_heads;
    if (!is_query && !write_kv) return;
    const int p = batch.positions[t], s = batch.token_seq[t];
    const int first = batch.cu_q[s];
    const int channels = per_token * dim;
    const float* ring = batch.state + (size_t)batch.slot_ids[s] * batch.state_stride + batch.state_offset;
    const int c0 = which * dim;                      // the head's first column of the row
    T* out;
    T* plain = nullptr;                              // where the head goes before rotation (the values that are the keys)
    if (is_query) {
        out = q_out + ((size_t)t * num_heads + which) * dim;
    } else {
        const int g = which - num_heads;
        const int block = block_table[(size_t)s * table_width + p / block_size];
        const size_t row = ((size_t)block * num_kv_heads + g) * block_size + (p % block_size);
        out = k_cache + row * dim;
        if (v_cache) plain = v_cache + row * dim;
    }
    const int half = rotated >> 1;
    if (interleaved && !(dim & 1) && !(row_stride & 1) && taps <= 8) {
        // a lane owns the pair (2i, 2i + 1): both numbers of every tap in one load, no number computed twice
        for (int pr = lane; pr < (dim >> 1); pr += 32) {
            const int c = c0 + 2 * pr;
            const float2 b = bias ? *(const float2*)(bias + c) : make_float2(0.0f, 0.0f);
            float2 sum;
            if (taps <= 1) {
                const float2 u = *(const float2*)(rows + (size_t)t * row_stride + c);
                sum = make_float2((u.x + b.x) * (taps == 1 ? conv_w[c] : 1.0f), (u.y + b.y) * (taps == 1 ? conv_w[c + 1] : 1.0f));
            } else {
                sum = make_float2(0.0f, 0.0f);
                for (int j = 0; j < taps; ++j) {
                    const int back = taps - 1 - j;
                    if (p - back < 0) continue;
                    float2 u;
                    if (t - back >= first) {
                        u = *(const float2*)(rows + (size_t)(t - back) * row_stride + c);
                        u.x += b.x; u.y += b.y;
                    } else {
                        const float* kept = ring + (size_t)((p - back) % taps) * channels + c;
                        u = make_float2(kept[0], kept[1]);
                    }
                    sum.x = fmaf(conv_w[(size_t)c * taps + j], u.x, sum.x);
                    sum.y = fmaf(conv_w[(size_t)(c + 1) * taps + j], u.y, sum.y);
                }
            }
            const int d = 2 * pr;
            if (plain) { plain[d] = from_float<T>(sum.x); plain[d + 1] = from_float<T>(sum.y); }
            float2 turned = sum;
            if (d < rotated) {
                const float2 cs = cos_sin[(size_t)p * half + pr];
                turned = make_float2(sum.x * cs.x - sum.y * cs.y, sum.y * cs.x + sum.x * cs.y);
            }
            out[d] = from_float<T>(turned.x);
            out[d + 1] = from_float<T>(turned.y);
        }
        return;
    }
    for (int d = lane; d < dim; d += 32) {
        const float mine = convolved(rows, row_stride, bias, conv_w, ring, channels, taps, t, p, first, c0 + d);
        if (plain) plain[d] = from_float<T>(mine);
        float value = mine;
        if (d < rotated) {
            const bool low = interleaved ? !(d & 1) : d < half;
            const int mate = interleaved ? (d ^ 1) : (low ? d + half : d - half);
            const int pair = interleaved ? (d >> 1) : (low ? d : d - half);
            const float other = convolved(rows, row_stride, bias, conv_w, ring, channels, taps, t, p, first, c0 + mate);
            const float2 cs = cos_sin[(size_t)p * half + pair];
            value = low ? mine * cs.x - other * cs.y : mine * cs.x + other * cs.y;
        }
        out[d] = from_float<T>(value);
    }
}

// grid (sequences, channel chunks): rows of the ring for the step's last taps - 1 positions of every sequence.
__global__ void __launch_bounds__(256)
short_conv_remember_kernel(const float* __restrict__ rows, int row_stride, const float* __restrict__ bias, int channels,
                           int taps, const ConvBatch batch) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int first = batch.cu_q[s], end = batch.cu_q[s + 1];
    float* ring = batch.state + (size_t)batch.slot_ids[s] * batch.state_stride + batch.state_offset;
    const float b = bias ? bias[c] : 0.0f;
    for (int t = max(first, end - (taps - 1)); t < end; ++t)
        ring[(size_t)(batch.positions[t] % taps) * channels + c] = rows[(size_t)t * row_stride + c] + b;
}

}  // namespace skv

using namespace skv;

// rows float [n, row_stride], normed in place: columns [offset, offset + width) of every row plus `bias`, divided by their
// root mean square (eps inside the root), times `weight`.  One or two segments (width_b 0: one).
SKV_EXPORT int skv_projection_norm(float* rows, int row_stride, int n, float eps, int offset_a, int width_a,
                                   const float* bias_a, const float* weight_a, int offset_b, int width_b,
                                   const float* bias_b, const float* weight_b, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!rows || width_a <= 0 || !weight_a || offset_a < 0 || offset_a + width_a > row_stride ||
        (width_b > 0 && (!weight_b || offset_b < 0 || offset_b + width_b > row_stride)))
        return fail("skv_projection_norm", "segments must lie inside a row and have weights");
    const NormSegment first{offset_a, width_a, bias_a, weight_a}, second{offset_b, width_b, bias_b, weight_b};
    return launch_pdl("skv_projection_norm", projection_norm_kernel, dim3(n, width_b > 0 ? 2 : 1), dim3(256), 0, stream,
                      rows, row_stride, eps, first, second);
}

static ConvBatch conv_batch(const int* positions, const int* token_seq, const int* cu_q, const int* slot_ids, float* state,
                            long long state_stride, long long state_offset) {
    ConvBatch batch;
    batch.positions = positions; batch.token_seq = token_seq; batch.cu_q = cu_q; batch.slot_ids = slot_ids;
    batch.state = state; batch.state_stride = state_stride; batch.state_offset = state_offset;
    return batch;
}

// rows float [n, row_stride]: [heads * dim queries | kv_heads * dim keys]; bias float [channels] or null; conv_w float
// [channels, taps] (taps 0: none); cos_sin float2 [positions, rotated / 2] or null with rotated 0; q_out [n, heads * dim],
// k_cache and v_cache [blocks, kv_heads, block_size, dim] in the compute dtype (v_cache null: the values are not the keys).
SKV_EXPORT int skv_short_conv_rotary(const float* rows, int row_stride, const float* bias, const float* conv_w, int taps,
                                     const float* cos_sin, int rotated, int interleaved, const int* block_table,
                                     int table_width, void* q_out, void* k_cache, void* v_cache, int n, int num_heads,
                                     int num_kv_heads, int dim, int block_size, int write_kv, const int* positions,
                                     const int* token_seq, const int* cu_q, const int* slot_ids, float* state,
                                     long long state_stride, long long state_offset, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (num_heads <= 0 || num_kv_heads <= 0 || dim <= 0 || block_size <= 0 || taps < 0 || rotated < 0 || rotated > dim ||
        (rotated & 1) || row_stride < (num_heads + num_kv_heads) * dim)
        return fail("skv_short_conv_rotary", "sizes do not agree");
    if (!rows || !q_out || !k_cache || !block_table || (taps > 0 && !conv_w) || (taps > 1 && !state) || (rotated > 0 && !cos_sin))
        return fail("skv_short_conv_rotary", "a pointer is missing");
    const long long items = (long long)n * (num_heads + num_kv_heads);
    return launch_pdl("skv_short_conv_rotary", short_conv_rotary_kernel<skv_t>, dim3((unsigned)((items + 7) / 8)), dim3(256),
                      0, stream, rows, row_stride, bias, conv_w, taps, (const float2*)cos_sin, rotated, interleaved,
                      block_table, table_width, (skv_t*)q_out, (skv_t*)k_cache, (skv_t*)v_cache, n, num_heads, num_kv_heads,
                      dim, block_size, write_kv, conv_batch(positions, token_seq, cu_q, slot_ids, state, state_stride, state_offset));
}

SKV_EXPORT int skv_short_conv_remember(const float* rows, int row_stride, const float* bias, int channels, int taps,
                                       int n_seqs, const int* positions, const int* token_seq, const int* cu_q,
                                       const int* slot_ids, float* state, long long state_stride, long long state_offset,
                                       cudaStream_t stream) {
    if (n_seqs <= 0 || taps <= 1) return 0;
    if (!rows || !state || channels <= 0 || row_stride < channels) return fail("skv_short_conv_remember", "sizes do not agree");
    return launch_pdl("skv_short_conv_remember", short_conv_remember_kernel, dim3(n_seqs, (channels + 255) / 256), dim3(256),
                      0, stream, rows, row_stride, bias, channels, taps,
                      conv_batch(positions, token_seq, cu_q, slot_ids, state, state_stride, state_offset));
}
