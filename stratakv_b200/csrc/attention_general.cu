// Attention with the head sizes as run-time arguments and the optional mechanisms that the
// head-size-specialised kernels do not have: biases on the projections, a norm on each value head,
// values narrower or wider than keys, a bias on the score that grows with the logarithm of the
// distance, and a gate per head on the output.  Two kernels:
//
//   qkv_finish:        float rows [q | k | v | ...] of the fused projection -> queries in the compute
//                      dtype, keys and (normalised) values in their places of the paged cache; a warp per
//                      (token, head);
//   attention_general: one warp per (token, head) over the sequence's own cached keys, online softmax
//                      by chunks of 32 keys, everything after the loads in float.
//
// score(i, j) = (q_i . k_j) * scale - r1[head] * ln(1 + r2[head] * (i - j))      (r1 null: no such term)
//               then cap * tanh(score / cap)                                      (cap 0: no cap)
// visible:      0 <= i - j < window   (window 0: every earlier key)
// out(i)      = softmax(score) . v  *  sigmoid(gate[i, head])                    (gate null: no gate; with
//               gate_per_element the logit of every output number: gate[i, head * vdim + d])
//
// qkv_finish can also divide every query and key head by its root mean square (unit norm, no weight, or with a
// weight on the keys, which is how a compressed latent per position is normed before it is cached), and multiply
// the queries of position p by 1 + coef * ln(floor((p + 1) / every) + 1).  A row may hold queries only (keys and
// values of another layer are used) or no values (vdim 0: the cached latent serves as key and value).
//
// Cache layout per entry: keys [block][kv_head][block_size][dim], values [block][kv_head][block_size][vdim].
// These kernels are the same in every build of the library (no compile-time head size); they serve the
// float32 path and every shape the specialised bfloat16 kernels do not take.
#include "common.cuh"

namespace skv {

constexpr int GEN_WARPS = 4;
constexpr int GEN_MAX_VDIM = 512;
constexpr int GEN_MERGE_ACC = GEN_MAX_VDIM / 32;   // what a lane of the merge keeps of a row of values                 // a lane keeps vdim / 32 accumulators: 8 up to 256, else 16

constexpr int FINISH_WARPS = 8;

// Optional steps of qkv_finish, all off when zero: the unit norm of query heads and of key heads (eps qk_eps; the
// keys' with a weight [kv_heads * dim] if k_weight is given) and the queries' temperature by position.
struct FinishExtras {
    int key_dim;               // width of a key head where it differs from a query head's (a cached latent); else dim
    int q_norm, k_norm;
    float qk_eps;
    const float* k_weight;
    float q_temp_coef;
    int q_temp_every;
};

template <typename T>
__device__ __forceinline__ void finish_store4(T* out, float4 v, float factor) {
    if (sizeof(T) == 4) {
        *(float4*)out = make_float4(v.x * factor, v.y * factor, v.z * factor, v.w * factor);
    } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * factor, v.y * factor);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * factor, v.w * factor);
        *(uint2*)out = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
    }
}

__device__ __forceinline__ float4 finish_load4(const float* x, const float* bias) {
    float4 v = *(const float4*)x;
    if (bias) {
        const float4 b = *(const float4*)bias;
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    }
    return v;
}

// One warp per (token, head): the token's query heads, then its key heads, then its value heads.
// value_norm != 0 divides each value head by sqrt(mean(v^2) + eps).  VEC: head sizes (at most 256) and the row
// stride are multiples of 4 and every pointer is 16-byte aligned; a lane then holds up to eight numbers of the
// head, whose loads go out before the lookups that say where the head is to be written.
template <typename T, bool VEC>
__global__ void __launch_bounds__(FINISH_WARPS * 32)
qkv_finish_kernel(const float* __restrict__ qkv, int row_stride, const float* __restrict__ q_bias,
                  const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                  const int* __restrict__ positions, const int* __restrict__ token_seq,
                  const int* __restrict__ block_table, int table_width, T* __restrict__ q_out,
                  T* __restrict__ k_cache, T* __restrict__ v_cache, int n_tokens, int num_heads, int num_kv_heads,
                  int dim, int vdim, int block_size, int value_norm, float value_eps, int write_kv,
                  const FinishExtras extras) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int per_token = num_heads + (vdim > 0 ? 2 : 1) * num_kv_heads;
    const long long item = (long long)blockIdx.x * FINISH_WARPS + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * per_token) return;        // whole warps leave together
    const int t = (int)(item / per_token), which = (int)(item - (long long)t * per_token);
    const bool is_query = which < num_heads, is_key = !is_query && which < num_heads + num_kv_heads;
    if (!is_query && !write_kv) return;
    const int g = is_query ? which : (is_key ? which - num_heads : which - num_heads - num_kv_heads);
    const int kdim = extras.key_dim;
    const int n = is_query ? dim : (is_key ? kdim : vdim);
    const float* x = qkv + (size_t)t * row_stride + (is_query ? (size_t)g * dim
                     : is_key ? (size_t)num_heads * dim + (size_t)g * kdim
                              : (size_t)num_heads * dim + (size_t)num_kv_heads * kdim + (size_t)g * vdim);
    const float* bias_base = is_query ? q_bias : (is_key ? k_bias : v_bias);
    const float* bias = bias_base ? bias_base + (size_t)g * n : nullptr;
    const bool normed = (!is_query && !is_key && value_norm) || (is_query && extras.q_norm) || (is_key && extras.k_norm);
    const float norm_eps = is_query || is_key ? extras.qk_eps : value_eps;
    const float* weight = is_key && extras.k_weight ? extras.k_weight + (size_t)g * n : nullptr;
    float temperature = 1.0f;
    if (is_query && extras.q_temp_every > 0)
        temperature = 1.0f + extras.q_temp_coef * logf((float)((positions[t] + 1) / extras.q_temp_every) + 1.0f);

    float4 held[2];
    if (VEC) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = 4 * lane + 128 * u;
            held[u] = i < n ? finish_load4(x + i, bias ? bias + i : nullptr) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
    T* out;
    if (is_query) {
        out = q_out + ((size_t)t * num_heads + g) * dim;
    } else {
        const int pos = positions[t];
        const int block = block_table[(size_t)token_seq[t] * table_width + pos / block_size];
        const size_t row = ((size_t)block * num_kv_heads + g) * block_size + (pos % block_size);
        out = (is_key ? k_cache : v_cache) + row * n;
    }
    float factor = 1.0f;
    if (VEC) {
        if (normed) {
            float squares = 0.0f;
#pragma unroll
            for (int u = 0; u < 2; ++u)
                squares += held[u].x * held[u].x + held[u].y * held[u].y + held[u].z * held[u].z + held[u].w * held[u].w;
            factor = 1.0f / sqrtf(warp_sum(squares) / (float)n + norm_eps);
        }
        factor *= temperature;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = 4 * lane + 128 * u;
            if (i < n) {
                if (weight) {
                    const float4 w4 = *(const float4*)(weight + i);
                    held[u].x *= w4.x; held[u].y *= w4.y; held[u].z *= w4.z; held[u].w *= w4.w;
                }
                finish_store4<T>(out + i, held[u], factor);
            }
        }
        return;
    }
    if (normed) {
        float squares = 0.0f;
        for (int d = lane; d < n; d += 32) {
            const float v = x[d] + (bias ? bias[d] : 0.0f);
            squares = fmaf(v, v, squares);
        }
        factor = 1.0f / sqrtf(warp_sum(squares) / (float)n + norm_eps);
    }
    factor *= temperature;
    for (int d = lane; d < n; d += 32)
        out[d] = from_float<T>((x[d] + (bias ? bias[d] : 0.0f)) * factor * (weight ? weight[d] : 1.0f));
}

// Rows of a paged cache with one head, copied into a plain matrix: out[i, :] = the row of position positions[i] of
// sequence seqs[i] (for a mixer that needs its sequences' cached vectors side by side, as a GEMM's input).
template <typename T>
__global__ void __launch_bounds__(256)
paged_gather_kernel(const T* __restrict__ cache, const int* __restrict__ block_table, int table_width,
                    const int* __restrict__ positions, const int* __restrict__ seqs, T* __restrict__ out, int n_rows,
                    int width, int block_size) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long i = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n_rows) return;
    const int pos = positions[i];
    const int block = block_table[(size_t)seqs[i] * table_width + pos / block_size];
    const T* from = cache + ((size_t)block * block_size + pos % block_size) * width;
    T* to = out + (size_t)i * width;
    for (int d = lane; d < width; d += 32) to[d] = from[d];
}

__device__ __forceinline__ float general_dot(const float* __restrict__ q, const float* __restrict__ row, int dim) {
    float sum = 0.0f;
    if ((dim & 3) == 0) {
        for (int d = 0; d < dim; d += 4) {
            const float4 k = *(const float4*)(row + d);
            sum = fmaf(q[d], k.x, sum); sum = fmaf(q[d + 1], k.y, sum);
            sum = fmaf(q[d + 2], k.z, sum); sum = fmaf(q[d + 3], k.w, sum);
        }
    } else {
        for (int d = 0; d < dim; ++d) sum = fmaf(q[d], row[d], sum);
    }
    return sum;
}

__device__ __forceinline__ float general_dot(const float* __restrict__ q, const __nv_bfloat16* __restrict__ row, int dim) {
    float sum = 0.0f;
    if ((dim & 7) == 0) {
        for (int d = 0; d < dim; d += 8) {
            const uint4 raw = *(const uint4*)(row + d);
            const __nv_bfloat162* pairs = (const __nv_bfloat162*)&raw;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 k = __bfloat1622float2(pairs[i]);
                sum = fmaf(q[d + 2 * i], k.x, sum);
                sum = fmaf(q[d + 2 * i + 1], k.y, sum);
            }
        }
    } else {
        for (int d = 0; d < dim; ++d) sum = fmaf(q[d], __bfloat162float(row[d]), sum);
    }
    return sum;
}

template <typename T, int GEN_ACC>
__global__ void __launch_bounds__(GEN_WARPS * 32)
attention_general_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int* __restrict__ block_table, int table_width, const int* __restrict__ positions,
                         const int* __restrict__ token_seq, T* __restrict__ out, int n_tokens, int num_heads,
                         int num_kv_heads, int dim, int vdim, int block_size, float scale, int window,
                         const float* __restrict__ r1, const float* __restrict__ r2, const float* __restrict__ gate,
                         int gate_stride, int out_stride, float softcap, int gate_per_element,
                         const float* __restrict__ sink, int v_stride, int splits, float* __restrict__ partial_o,
                         float* __restrict__ partial_ml) {
    extern __shared__ __align__(16) float general_q[];          // [GEN_WARPS][dim rounded up to 4]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long work = (long long)blockIdx.x * GEN_WARPS + warp;
    if (work >= (long long)n_tokens * num_heads * splits) return;        // whole warps leave together
    // With splits > 1 a warp takes one part of its (token, head)'s keys and leaves its sums, their maximum and its
    // unnormalised output for attention_general_merge_kernel; the heads of a token stay side by side in a block.
    const long long item = splits > 1 ? (work / ((long long)num_heads * splits)) * num_heads + work % num_heads : work;
    const int split = splits > 1 ? (int)((work / num_heads) % splits) : 0;
    const int t = (int)(item / num_heads), head = (int)(item % num_heads);
    const int kv_head = head / (num_heads / num_kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)token_seq[t] * table_width;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const float slope = r1 ? r1[head] : 0.0f, reach = r1 ? r2[head] : 0.0f;

    float* qs = general_q + (size_t)warp * ((dim + 3) & ~3);
    const T* q_row = q + ((size_t)t * num_heads + head) * dim;
    for (int d = lane; d < dim; d += 32) qs[d] = to_float(q_row[d]);
    __syncwarp();

    float acc[GEN_ACC];
#pragma unroll
    for (int i = 0; i < GEN_ACC; ++i) acc[i] = 0.0f;
    float running_max = -INFINITY, running_sum = 0.0f;

    // this warp's keys: all of lo .. pos, or its part of them in whole runs of 32
    int first_key = lo, last_key = pos;
    if (splits > 1) {
        const int runs = (pos - lo + 32) / 32, per_split = (runs + splits - 1) / splits;
        first_key = lo + split * per_split * 32;
        last_key = min(pos, first_key + per_split * 32 - 1);
    }
    for (int j0 = first_key; j0 <= last_key; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= last_key;
        size_t row = 0;                                // row of this key in units of one head's vector
        float score = -INFINITY;
        if (valid) {
            const int block = table[j / block_size];
            row = ((size_t)block * num_kv_heads + kv_head) * block_size + (j % block_size);
            score = general_dot(qs, k_cache + row * dim, dim) * scale;
            if (r1) score -= slope * log1pf(reach * (float)(pos - j));
            if (softcap > 0.0f) score = softcap * tanhf(score / softcap);
        }
        const float new_max = fmaxf(running_max, warp_max(score));
        const float p = valid ? expf(score - new_max) : 0.0f;
        const float rescale = expf(running_max - new_max);     // 0 on the first chunk
        running_sum = running_sum * rescale + warp_sum(p);
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < GEN_ACC; ++i) acc[i] *= rescale;
        const int count = min(32, last_key - j0 + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
            const T* v_row = v_cache + (size_t)rj * v_stride;
#pragma unroll
            for (int i = 0; i < GEN_ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < vdim) acc[i] = fmaf(pj, to_float(v_row[d]), acc[i]);
            }
        }
    }
    if (splits > 1) {
        float* o_part = partial_o + ((size_t)item * splits + split) * vdim;
#pragma unroll
        for (int i = 0; i < GEN_ACC; ++i) {
            const int d = lane + 32 * i;
            if (d < vdim) o_part[d] = acc[i];
        }
        if (lane == 0) {
            partial_ml[((size_t)item * splits + split) * 2] = running_max;      // -infinity: this part had no keys
            partial_ml[((size_t)item * splits + split) * 2 + 1] = running_sum;
        }
        return;
    }
    // a sink counts once in the denominator: it has no key and no value, and is not scaled
    if (sink) running_sum += expf(sink[head] - running_max);
    float factor = 1.0f / running_sum;
    if (gate && !gate_per_element) factor *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + head]));
    const float* gate_row = gate && gate_per_element ? gate + (size_t)t * gate_stride + (size_t)head * vdim : nullptr;
    T* out_row = out + (size_t)t * out_stride + (size_t)head * vdim;
#pragma unroll
    for (int i = 0; i < GEN_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) {
            float value = acc[i] * factor;
            if (gate_row) value *= 1.0f / (1.0f + expf(-gate_row[d]));
            out_row[d] = from_float<T>(value);
        }
    }
    // columns that pad a row for the projection after it are zero
    if (head == num_heads - 1)
        for (int c = num_heads * vdim + lane; c < out_stride; c += 32) out[(size_t)t * out_stride + c] = from_float<T>(0.0f);
}

// The parts of a (token, head) that attention_general_kernel left with splits > 1, put together: the largest maximum,
// the sums and outputs brought to it, the sink, the gate.  A warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(GEN_WARPS * 32)
attention_general_merge_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                               T* __restrict__ out, int n_tokens, int num_heads, int vdim, int splits,
                               const float* __restrict__ gate, int gate_stride, int out_stride, int gate_per_element,
                               const float* __restrict__ sink) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * GEN_WARPS + warp;
    if (item >= (long long)n_tokens * num_heads) return;
    const int t = (int)(item / num_heads), head = (int)(item % num_heads);
    const float* ml = partial_ml + (size_t)item * splits * 2;
    // lane s (and s + 32, ...) holds part s's maximum and sum; the weights exp(max_s - top) are made once
    float top = -INFINITY;
    for (int s = lane; s < splits; s += 32) top = fmaxf(top, ml[2 * s]);      // (the first part always has the first key)
    top = warp_max(top);
    float total = 0.0f;
    for (int s = lane; s < splits; s += 32) total += ml[2 * s] == -INFINITY ? 0.0f : ml[2 * s + 1] * expf(ml[2 * s] - top);
    total = warp_sum(total);
    if (sink) total += expf(sink[head] - top);
    float factor = 1.0f / total;
    if (gate && !gate_per_element) factor *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + head]));
    const float* gate_row = gate && gate_per_element ? gate + (size_t)t * gate_stride + (size_t)head * vdim : nullptr;
    T* out_row = out + (size_t)t * out_stride + (size_t)head * vdim;
    const float* o_parts = partial_o + (size_t)item * splits * vdim;
    float value[GEN_MERGE_ACC];
#pragma unroll
    for (int i = 0; i < GEN_MERGE_ACC; ++i) value[i] = 0.0f;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        const int mine = s0 + lane;
        const float m = mine < splits ? ml[2 * mine] : -INFINITY;
        const float weight = m == -INFINITY ? 0.0f : expf(m - top) * factor;
        const int count = min(32, splits - s0);
        for (int j = 0; j < count; ++j) {
            const float w = __shfl_sync(0xffffffffu, weight, j);
            if (w == 0.0f) continue;                                   // (a part without keys left nothing to read)
            const float* part = o_parts + (size_t)(s0 + j) * vdim;
#pragma unroll
            for (int i = 0; i < GEN_MERGE_ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < vdim) value[i] = fmaf(part[d], w, value[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < GEN_MERGE_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < vdim) {
            float v = value[i];
            if (gate_row) v *= 1.0f / (1.0f + expf(-gate_row[d]));
            out_row[d] = from_float<T>(v);
        }
    }
    if (head == num_heads - 1)
        for (int c = num_heads * vdim + lane; c < out_stride; c += 32) out[(size_t)t * out_stride + c] = from_float<T>(0.0f);
}

}  // namespace skv

using namespace skv;

// `qkv`: float [n_tokens, row_stride], a row holding heads*dim query, kv_heads*dim key and kv_heads*vdim value
// numbers (whatever follows them is not read).  Biases are float and may be null.
SKV_EXPORT int skv_qkv_finish(const float* qkv, int row_stride, const float* q_bias, const float* k_bias,
                              const float* v_bias, const int* positions, const int* token_seq,
                              const int* block_table, int table_width, void* q_out, void* k_cache, void* v_cache,
                              int n_tokens, int num_heads, int num_kv_heads, int dim, int vdim, int block_size,
                              int value_norm, float value_eps, int write_kv, int q_norm, int k_norm, float qk_eps,
                              const float* k_weight, float q_temp_coef, int q_temp_every, int key_dim,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (num_heads < 0 || num_kv_heads <= 0 || dim <= 0 || vdim < 0 || block_size <= 0 || (num_heads > 0 && !q_out))
        return fail("skv_qkv_finish", "head counts, head sizes and block_size must be positive");
    if (key_dim <= 0) key_dim = dim;
    if (row_stride < (write_kv ? num_heads * dim + num_kv_heads * (key_dim + vdim) : num_heads * dim))
        return fail("skv_qkv_finish", "a row is shorter than its queries, keys and values");
    if (q_temp_every < 0) return fail("skv_qkv_finish", "the temperature's period must not be negative");
    const FinishExtras extras = {key_dim, q_norm, k_norm, qk_eps, k_weight, q_temp_coef, q_temp_every};
    const long long items = (long long)n_tokens * (num_heads + (vdim > 0 ? 2 : 1) * num_kv_heads);
    const long long blocks = (items + FINISH_WARPS - 1) / FINISH_WARPS;
    if (blocks > 0x7fffffffLL) return fail("skv_qkv_finish", "too many tokens in one step");
    const bool vec = dim % 4 == 0 && vdim % 4 == 0 && key_dim % 4 == 0 && dim <= 256 && vdim <= 256 && key_dim <= 256 &&
                     row_stride % 4 == 0 &&
                     (((uintptr_t)qkv | (uintptr_t)q_bias | (uintptr_t)k_bias | (uintptr_t)v_bias | (uintptr_t)q_out |
                       (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)k_weight) & 15) == 0;
    auto kernel = vec ? qkv_finish_kernel<skv_t, true> : qkv_finish_kernel<skv_t, false>;
    return launch_pdl("skv_qkv_finish", kernel, dim3((unsigned)blocks), dim3(FINISH_WARPS * 32), 0, stream, qkv,
                      row_stride, q_bias, k_bias, v_bias, positions, token_seq, block_table, table_width,
                      (skv_t*)q_out, (skv_t*)k_cache, (skv_t*)v_cache, n_tokens, num_heads, num_kv_heads, dim, vdim,
                      block_size, value_norm, value_eps, write_kv, extras);
}

// cache: [blocks][1][block_size][width] in the compute dtype; out [n_rows, width].
SKV_EXPORT int skv_paged_gather(const void* cache, const int* block_table, int table_width, const int* positions,
                                const int* seqs, void* out, int n_rows, int width, int block_size, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || block_size <= 0 || table_width <= 0) return fail("skv_paged_gather", "sizes must be positive");
    return launch_pdl("skv_paged_gather", paged_gather_kernel<skv_t>, dim3((n_rows + 7) / 8), dim3(256), 0, stream,
                      (const skv_t*)cache, block_table, table_width, positions, seqs, (skv_t*)out, n_rows, width, block_size);
}

// `r1`, `r2`: float [num_heads] or both null.  `gate`: float, the gate's logit of (token t, head h) at
// gate[t * gate_stride + h], or null.  `out` rows are out_stride >= heads * vdim apart; what lies beyond a row's
// heads is set to zero.  `sink`: float [num_heads] or null; exp(sink[h]) is added to the softmax's denominator.
// `value_stride`: numbers between the values' rows (0: vdim), so that the head of a wider cached row can be the value.
SKV_EXPORT int skv_attention_general(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                     int table_width, const int* positions, const int* token_seq, void* out,
                                     int n_tokens, int num_heads, int num_kv_heads, int dim, int vdim, int block_size,
                                     float scale, int window, const float* r1, const float* r2, const float* gate,
                                     int gate_stride, int out_stride, float softcap, int gate_per_element,
                                     const float* sink, int value_stride, int splits, float* partial_o,
                                     float* partial_ml, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (splits < 1 || splits > 1024 || (splits > 1 && (!partial_o || !partial_ml)))
        return fail("skv_attention_general", "1 to 1024 parts of the keys, and with more than one the scratch for them");
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail("skv_attention_general", "heads must be a positive multiple of kv heads");
    if (dim <= 0 || vdim <= 0 || vdim > GEN_MAX_VDIM) return fail("skv_attention_general", "value heads of 1 to 512 numbers are served");
    if (softcap < 0.0f) return fail("skv_attention_general", "the cap on the scores must not be negative");
    if (value_stride <= 0) value_stride = vdim;
    if (value_stride < vdim) return fail("skv_attention_general", "the values' rows cannot be closer together than they are wide");
    if (block_size <= 0 || window < 0) return fail("skv_attention_general", "bad block size or window");
    if (out_stride < num_heads * vdim) return fail("skv_attention_general", "a row of the output is shorter than its heads");
    if ((r1 == nullptr) != (r2 == nullptr)) return fail("skv_attention_general", "the distance bias needs both of its numbers per head");
    const size_t smem = (size_t)GEN_WARPS * ((dim + 3) & ~3) * sizeof(float);
    if (smem > 48 * 1024) return fail("skv_attention_general", "the key size is too large");
    const long long items = (long long)n_tokens * num_heads;
    const long long blocks = (items * splits + GEN_WARPS - 1) / GEN_WARPS;
    if (blocks > 0x7fffffffLL) return fail("skv_attention_general", "too many tokens in one step");
    auto kernel = vdim <= 256 ? attention_general_kernel<skv_t, 8> : attention_general_kernel<skv_t, 16>;
    if (int code = launch_pdl("skv_attention_general", kernel, dim3((unsigned)blocks),
                              dim3(GEN_WARPS * 32), smem, stream, (const skv_t*)q, (const skv_t*)k_cache,
                              (const skv_t*)v_cache, block_table, table_width, positions, token_seq, (skv_t*)out, n_tokens,
                              num_heads, num_kv_heads, dim, vdim, block_size, scale, window, r1, r2, gate, gate_stride,
                              out_stride, softcap, gate_per_element, sink, value_stride, splits, partial_o, partial_ml))
        return code;
    if (splits == 1) return 0;
    return launch_pdl("skv_attention_general(merge)", attention_general_merge_kernel<skv_t>,
                      dim3((unsigned)((items + GEN_WARPS - 1) / GEN_WARPS)), dim3(GEN_WARPS * 32), 0, stream,
                      (const float*)partial_o, (const float*)partial_ml, (skv_t*)out, n_tokens, num_heads, vdim, splits,
                      gate, gate_stride, out_stride, gate_per_element, sink);
}
