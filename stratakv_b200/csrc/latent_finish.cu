// What follows the fused projection of a latent-attention layer whose queries and keys have a rotated part.
//
// A float row of the projection holds, per head, `dim` unrotated and `rope_dim` rotated query numbers, and (for a layer
// with a cache of its own, at latent_offset) `latent_dim` numbers of the compressed vector and `rope_dim` numbers of
// the one key part that all heads share.  Per token, a block
//   - copies the unrotated query parts to q_plain [tokens, heads * dim] (the keys' up-projection is folded into them
//     by the per-head product that follows),
//   - rotates the rotated query parts and puts them behind the (not yet written) folded part of every head of
//     q_folded [tokens, heads * (latent_dim + rope_dim)]
//     (or, where the step makes every head's keys instead of folding: both parts, head by head, to
//     q_whole [tokens, heads * (dim + rope_dim)], and nothing to the other two),
//   - divides the compressed vector by its root mean square, multiplies by the norm's weight, rotates the key part,
//     and writes both into the token's row of the paged cache [blocks][1][block_size][latent_dim + rope_dim].
// Rotation: of the first `rotated` numbers of a part, number i is paired with number i + rotated/2;
// (u, v) -> (u cos - v sin, v cos + u sin) with (cos, sin) = table[position][i].  Float math; the outputs are rounded
// to the compute dtype.
#include "common.cuh"

namespace skv {

constexpr int LATENT_FINISH_THREADS = 256;

// The value of number r of a part x after the rotation (r < part width).
__device__ __forceinline__ float turned(const float* x, int r, int rotated, const float* cos_sin) {
    if (r >= rotated) return x[r];
    const int half = rotated >> 1;
    if (r < half) return x[r] * cos_sin[2 * r] - x[r + half] * cos_sin[2 * r + 1];
    const int i = r - half;
    return x[r] * cos_sin[2 * i] + x[i] * cos_sin[2 * i + 1];
}

template <typename T>
__global__ void __launch_bounds__(LATENT_FINISH_THREADS)
latent_finish_kernel(const float* __restrict__ fused, int row_stride, T* __restrict__ q_plain, T* __restrict__ q_folded,
                     T* __restrict__ q_whole, T* __restrict__ cache, const int* __restrict__ positions, const int* __restrict__ token_seq,
                     const int* __restrict__ block_table, int table_width, int heads, int dim, int rope_dim,
                     int latent_dim, int block_size, const float* __restrict__ rotation, int rotated, int table_len,
                     int latent_offset, const float* __restrict__ latent_gamma, float eps, int write_cache) {
    __shared__ float reduce[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = fused + (size_t)t * row_stride;
    const int pos = positions[t];
    const float* cos_sin = rotation ? rotation + (size_t)min(pos, table_len - 1) * rotated : nullptr;
    const int turn = rotation ? rotated : 0;
    const int q_head = dim + rope_dim, key_dim = latent_dim + rope_dim;
    for (int idx = threadIdx.x; idx < heads * q_head; idx += LATENT_FINISH_THREADS) {
        const int head = idx / q_head, j = idx - head * q_head;
        const float value = j < dim ? row[idx] : turned(row + (size_t)head * q_head + dim, j - dim, turn, cos_sin);
        if (q_whole) q_whole[(size_t)t * heads * q_head + idx] = from_float<T>(value);
        else if (j < dim) q_plain[((size_t)t * heads + head) * dim + j] = from_float<T>(value);
        else q_folded[((size_t)t * heads + head) * key_dim + latent_dim + (j - dim)] = from_float<T>(value);
    }
    if (!write_cache) return;
    const float* latent = row + latent_offset;
    float squares = 0.0f;
    for (int j = threadIdx.x; j < latent_dim; j += LATENT_FINISH_THREADS) squares = fmaf(latent[j], latent[j], squares);
    const float factor = 1.0f / sqrtf(block_sum(squares, reduce) / (float)latent_dim + eps);
    const int block = block_table[(size_t)token_seq[t] * table_width + pos / block_size];
    T* out = cache + ((size_t)block * block_size + pos % block_size) * key_dim;
    for (int j = threadIdx.x; j < key_dim; j += LATENT_FINISH_THREADS) {
        const float value = j < latent_dim ? latent[j] * factor * latent_gamma[j]
                                           : turned(latent + latent_dim, j - latent_dim, turn, cos_sin);
        out[j] = from_float<T>(value);
    }
}

}  // namespace skv

using namespace skv;

// q_whole: null, or the one place for the queries (then q_plain and q_folded may be null).
// rotation: float [table_len][rotated / 2][2] or null (then nothing is rotated).  With write_cache 0 a row need hold
// its queries only, and latent_gamma may be null.
SKV_EXPORT int skv_latent_finish(const float* fused, int row_stride, void* q_plain, void* q_folded, void* q_whole, void* cache,
                                 const int* positions, const int* token_seq, const int* block_table, int table_width,
                                 int n_tokens, int heads, int dim, int rope_dim, int latent_dim, int block_size,
                                 const float* rotation, int rotated, int table_len, int latent_offset,
                                 const float* latent_gamma, float eps, int write_cache, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (heads <= 0 || dim <= 0 || rope_dim < 0 || latent_dim <= 0 || block_size <= 0)
        return fail("skv_latent_finish", "head count, sizes and block_size must be positive");
    if (rotation && (rotated <= 0 || rotated % 2 || rotated > rope_dim || table_len <= 0))
        return fail("skv_latent_finish", "the rotated numbers must be an even count within the rotated part");
    if (!fused || (!q_whole && (!q_plain || !q_folded)))
        return fail("skv_latent_finish", "a place for the queries is needed: the two parts apart, or whole heads");
    if (write_cache && (!latent_gamma || !cache || latent_offset < heads * (dim + rope_dim)))
        return fail("skv_latent_finish", "a cache write needs the cache, the latent's norm weight and the latent behind the queries");
    if (row_stride < (write_cache ? latent_offset + latent_dim + rope_dim : heads * (dim + rope_dim)))
        return fail("skv_latent_finish", "a row is shorter than its queries, latent and key part");
    return launch_pdl("skv_latent_finish", latent_finish_kernel<skv_t>, dim3(n_tokens), dim3(LATENT_FINISH_THREADS), 0,
                      stream, fused, row_stride, (skv_t*)q_plain, (skv_t*)q_folded, (skv_t*)q_whole, (skv_t*)cache, positions, token_seq,
                      block_table, table_width, heads, dim, rope_dim, latent_dim, block_size, rotation,
                      rotation ? rotated : 0, table_len, latent_offset, latent_gamma, eps, write_cache);
}
