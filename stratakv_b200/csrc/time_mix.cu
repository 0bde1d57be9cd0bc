// Time mixing with a matrix state per head and a decay per token and key channel (the RWKV family's mixer), over packed
// steps of several sequences.  For a sequence's token at position p, with h' the token before's input (zeros at p = 0):
//
//   mix_s = h + (h' - h) * mu_s                     one mix per projection s (token_shift_mix)
//   r, k, v, gate logits, decay logits               the library's projections of those mixes
//   w     = exp(-exp(W2 tanh(lora) + w0))            time_mix_decay; lora = W1 mix_w
//   o_p   = (S_(p-1) + diag(u) k_p v_p^T)^T r_p      time_mix_scan; S is [key channel][value channel] per head
//   S_p   = diag(w_p) S_(p-1) + k_p v_p^T
//   out_p = o_p / rms(o_p) per head * norm * silu(gate) * out_scale      time_mix_finish (compute dtype: the input of
//                                                                        the output projection)
//
// Everything between the projections is float.  Per sequence the cache keeps float state, one row per slot, starting
// `state_offset` floats into the row:
//   [2][heads][dim][dim]  S after the sequence's last position, in the half chosen by that position's parity: a step
//                         reads the half of the position before its first token and writes the half of its last, so a
//                         one-token step that runs twice (a graph's capture after its warm-up) computes the same thing;
//   [2][hidden]           the mixer's input at the last position, by the same rule.  token_shift_mix reads it and the
//                         scan, which runs later in the same step, writes it: no kernel reads what it writes.
// A sequence's first token (position 0) ignores the state, so a slot's earlier user leaves nothing behind.
#include "common.cuh"

namespace skv {

struct TimeMixBatch {
    const int* positions;      // [tokens]
    const int* token_seq;      // [tokens]
    const int* cu_q;           // [seqs + 1]
    const int* slot_ids;       // [seqs]
    float* state;              // [slots][state_stride] floats
    long long state_stride;    // floats per slot
    long long state_offset;    // where this mixer's state starts within a slot's row
};

constexpr int TM_MAX_MIXES = 8;
constexpr int TM_REGS = 16;            // key channels of one value column that a thread of the scan keeps (or 4)

// Eight neighbouring numbers of a row, as floats (16 bytes of bfloat16 or 32 of float at a time).
__device__ __forceinline__ void tm_load8(const float* p, float* v) {
    const float4 a = ((const float4*)p)[0], b = ((const float4*)p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void tm_load8(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *(const uint4*)p;
    const __nv_bfloat162* pairs = (const __nv_bfloat162*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(pairs[i]);
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void tm_store8(float* p, const float* v) {
    ((float4*)p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    ((float4*)p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void tm_store8(__nv_bfloat16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* pairs = (__nv_bfloat162*)&raw;
#pragma unroll
    for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *(uint4*)p = raw;
}

// mixes[s][t][c] = h[t][c] + (before[t][c] - h[t][c]) * mu[s][c]; a block per token, threads over the channels (VEC: eight
// channels a thread where the width is a multiple of 8 and the rows are 16-byte aligned).
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
token_shift_mix_kernel(const T* __restrict__ h, const float* __restrict__ mu, T* __restrict__ mixes, int n_tokens,
                       int hidden, int n_mixes, long long before_offset, const TimeMixBatch batch) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int p = batch.positions[t], s = batch.token_seq[t];
    const bool inside = t > batch.cu_q[s];
    const float* kept = batch.state + (size_t)batch.slot_ids[s] * batch.state_stride + batch.state_offset + before_offset +
                        (size_t)((p - 1) & 1) * hidden;
    if (VEC) {
        for (int c = 8 * threadIdx.x; c < hidden; c += 8 * blockDim.x) {
            float now[8], before[8], factor[8], mixed[8];
            tm_load8(h + (size_t)t * hidden + c, now);
            if (inside) {
                tm_load8(h + (size_t)(t - 1) * hidden + c, before);
            } else if (p > 0) {
                tm_load8(kept + c, before);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) before[i] = 0.0f;
            }
            for (int m = 0; m < n_mixes; ++m) {
                tm_load8(mu + (size_t)m * hidden + c, factor);
#pragma unroll
                for (int i = 0; i < 8; ++i) mixed[i] = fmaf(before[i] - now[i], factor[i], now[i]);
                tm_store8(mixes + ((size_t)m * n_tokens + t) * hidden + c, mixed);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float now = to_float(h[(size_t)t * hidden + c]);
        const float before = inside ? to_float(h[(size_t)(t - 1) * hidden + c]) : (p > 0 ? kept[c] : 0.0f);
        const float delta = before - now;
        for (int m = 0; m < n_mixes; ++m)
            mixes[((size_t)m * n_tokens + t) * hidden + c] = from_float<T>(fmaf(delta, mu[(size_t)m * hidden + c], now));
    }
}

// decay[t][c] = exp(-exp(w0[c] + sum_j w2t[j][c] * tanh(lora[t][j]))); a block per TM_DECAY_TOKENS tokens and 256
// channels, a thread a channel (w2t is the weight transposed, [rank][channels], so that neighbouring threads read neighbouring numbers
// and a number that is read serves all of the block's tokens).
constexpr int TM_DECAY_TOKENS = 4;
template <typename T>
__global__ void __launch_bounds__(256)
time_mix_decay_kernel(const float* __restrict__ lora, int lora_stride, int rank, const T* __restrict__ w2t,
                      const float* __restrict__ w0, float* __restrict__ decay, int n_tokens, int channels) {
    extern __shared__ __align__(16) float tm_lora[];          // [TM_DECAY_TOKENS][rank]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * TM_DECAY_TOKENS;
    const int count = min(TM_DECAY_TOKENS, n_tokens - t0);
    for (int idx = threadIdx.x; idx < TM_DECAY_TOKENS * rank; idx += blockDim.x) {
        const int tok = idx / rank, j = idx - tok * rank;
        tm_lora[idx] = tok < count ? tanhf(lora[(size_t)(t0 + tok) * lora_stride + j]) : 0.0f;
    }
    __syncthreads();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c < channels) {
        float z[TM_DECAY_TOKENS];
#pragma unroll
        for (int tok = 0; tok < TM_DECAY_TOKENS; ++tok) z[tok] = w0[c];
        for (int j = 0; j < rank; ++j) {
            const float w = to_float(w2t[(size_t)j * channels + c]);
#pragma unroll
            for (int tok = 0; tok < TM_DECAY_TOKENS; ++tok) z[tok] = fmaf(w, tm_lora[tok * rank + j], z[tok]);
        }
#pragma unroll
        for (int tok = 0; tok < TM_DECAY_TOKENS; ++tok)
            if (tok < count) decay[(size_t)(t0 + tok) * channels + c] = expf(-expf(z[tok]));
    }
}

__device__ __forceinline__ void tm_copy_async(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

// The recurrence.  A block per (sequence, head, slice of value columns); thread (column c, part s of `key_split`) keeps
// S[i][c] for the TM_REGS key channels i = s * TM_REGS ..; the tokens' r, k, w (the whole head) and v (the block's
// columns) are staged in shared memory a few tokens at a time, the next tokens' copies on their way while these are
// worked on.  A part's TM_REGS channels lie TM_PART_STRIDE floats from the next part's, so that the four parts a quarter
// of a warp reads at once fall into different banks; channels past the head's last stay zero.  A thread fetches the
// next token's numbers from shared memory before it works on this token's.  The head-0 block of a sequence's first
// slice also remembers the mixer's input at the sequence's last token.
// REGS is 16 where a step has blocks enough to fill the GPU, and 4 where it has not (one prompt alone): a thread then
// has a quarter of the sums to make one after the other and a warp's shuffles bring four times as many together.
template <int REGS> struct TimeMixLayout { static constexpr int stride = REGS == 16 ? 20 : REGS; };

template <int REGS>
struct TimeMixToken {
    float4 r[REGS / 4], k[REGS / 4], w[REGS / 4];
    float v;
};

template <int REGS>
__device__ __forceinline__ void tm_fetch(TimeMixToken<REGS>& token, const float* sr, const float* sk, const float* sw,
                                         const float* sv, int row, int column, bool active) {
#pragma unroll
    for (int q = 0; q < REGS / 4; ++q) {
        token.r[q] = ((const float4*)(sr + row))[q];
        token.k[q] = ((const float4*)(sk + row))[q];
        token.w[q] = ((const float4*)(sw + row))[q];
    }
    token.v = active ? sv[column] : 0.0f;
}

template <typename T, int REGS>
__global__ void __launch_bounds__(256)
time_mix_scan_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                     const float* __restrict__ decay, int stride, const float* __restrict__ bonus,
                     float* __restrict__ out, const T* __restrict__ h, int hidden, int heads, int dim, int key_split,
                     int cols, int chunk, const TimeMixBatch batch) {
    extern __shared__ __align__(16) float tm_stage[];
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
    const int first = batch.cu_q[seq], n = batch.cu_q[seq + 1] - first;
    if (n <= 0) return;
    const int p0 = batch.positions[first];
    float* slot_state = batch.state + (size_t)batch.slot_ids[seq] * batch.state_stride + batch.state_offset;
    const size_t half = (size_t)heads * dim * dim;
    const float* s_read = slot_state + (size_t)((p0 - 1) & 1) * half + (size_t)head * dim * dim;
    float* s_write = slot_state + (size_t)((p0 + n - 1) & 1) * half + (size_t)head * dim * dim;
    const int part = threadIdx.x % key_split, c = threadIdx.x / key_split, col = col0 + c;
    const bool active = c < cols && col < dim;
    const int padded = key_split * TimeMixLayout<REGS>::stride;
    float S[REGS], u[REGS];
#pragma unroll
    for (int j = 0; j < REGS; ++j) {
        const int i = part * REGS + j;
        const bool held = active && i < dim;
        S[j] = held && p0 > 0 ? s_read[(size_t)i * dim + col] : 0.0f;
        u[j] = held ? bonus[(size_t)head * dim + i] : 0.0f;
    }
    // two sets of buffers, each [chunk][padded] for r, k, w and [chunk][cols] for v
    const int set = chunk * (3 * padded + cols);
    for (int idx = threadIdx.x; idx < 2 * set; idx += blockDim.x) tm_stage[idx] = 0.0f;      // (the padding stays zero)
    __syncthreads();

    auto stage = [&](int which, int t0) {
        float* sr = tm_stage + which * set;
        float* sk = sr + chunk * padded;
        float* sw = sk + chunk * padded;
        float* sv = sw + chunk * padded;
        const int m = min(chunk, n - t0);
        for (int idx = threadIdx.x; idx < m * dim; idx += blockDim.x) {
            const int tok = idx / dim, i = idx - tok * dim;
            const size_t at = (size_t)(first + t0 + tok) * stride + (size_t)head * dim + i;
            const int to = tok * padded + (i / REGS) * TimeMixLayout<REGS>::stride + (i % REGS);
            tm_copy_async(sr + to, r + at);
            tm_copy_async(sk + to, k + at);
            tm_copy_async(sw + to, decay + at);
        }
        const int width = min(cols, dim - col0);
        for (int idx = threadIdx.x; idx < m * width; idx += blockDim.x) {
            const int tok = idx / width, j = idx - tok * width;
            tm_copy_async(sv + tok * cols + j, v + (size_t)(first + t0 + tok) * stride + (size_t)head * dim + col0 + j);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    stage(0, 0);
    int which = 0;
    for (int t0 = 0; t0 < n; t0 += chunk, which ^= 1) {
        const bool more = t0 + chunk < n;
        if (more) {
            stage(which ^ 1, t0 + chunk);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* sr = tm_stage + which * set;
        const float* sk = sr + chunk * padded;
        const float* sw = sk + chunk * padded;
        const float* sv = sw + chunk * padded;
        const int m = min(chunk, n - t0);
        const int mine = part * TimeMixLayout<REGS>::stride;
        float* to = out + (size_t)(first + t0) * stride + (size_t)head * dim + col;
        // one token: its share of o (summed over the parts by shuffles) and the new S
        auto work = [&](const TimeMixToken<REGS>& now) {
            const float vj = now.v;
            float acc = 0.0f;
#pragma unroll
            for (int q = 0; q < REGS / 4; ++q) {
                const float4 r4 = now.r[q], k4 = now.k[q], w4 = now.w[q];
                float kv;
                kv = k4.x * vj; acc = fmaf(r4.x, fmaf(u[4 * q], kv, S[4 * q]), acc); S[4 * q] = fmaf(w4.x, S[4 * q], kv);
                kv = k4.y * vj; acc = fmaf(r4.y, fmaf(u[4 * q + 1], kv, S[4 * q + 1]), acc); S[4 * q + 1] = fmaf(w4.y, S[4 * q + 1], kv);
                kv = k4.z * vj; acc = fmaf(r4.z, fmaf(u[4 * q + 2], kv, S[4 * q + 2]), acc); S[4 * q + 2] = fmaf(w4.z, S[4 * q + 2], kv);
                kv = k4.w * vj; acc = fmaf(r4.w, fmaf(u[4 * q + 3], kv, S[4 * q + 3]), acc); S[4 * q + 3] = fmaf(w4.w, S[4 * q + 3], kv);
            }
            for (int offset = key_split >> 1; offset > 0; offset >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, offset);
            if (part == 0 && active) *to = acc;
            to += stride;
        };
        // two tokens a round, each fetched from shared memory while the other is worked on
        TimeMixToken<REGS> even, odd;
        tm_fetch(even, sr, sk, sw, sv, mine, c, active);
        for (int tok = 0; tok < m; tok += 2) {
            if (tok + 1 < m) tm_fetch(odd, sr, sk, sw, sv, (tok + 1) * padded + mine, (tok + 1) * cols + c, active);
            work(even);
            if (tok + 1 < m) {
                if (tok + 2 < m) tm_fetch(even, sr, sk, sw, sv, (tok + 2) * padded + mine, (tok + 2) * cols + c, active);
                work(odd);
            }
        }
        __syncthreads();                            // before the next round's copies land in this set
    }
#pragma unroll
    for (int j = 0; j < REGS; ++j) {
        const int i = part * REGS + j;
        if (active && i < dim) s_write[(size_t)i * dim + col] = S[j];
    }
    if (head == 0 && blockIdx.z == 0) {
        float* kept = slot_state + 2 * half + (size_t)((p0 + n - 1) & 1) * hidden;
        const T* last = h + (size_t)(first + n - 1) * hidden;
        for (int w = threadIdx.x; w < hidden; w += blockDim.x) kept[w] = to_float(last[w]);
    }
}

// out[t][head] = o / rms(o) * norm * silu(gate) * out_scale; a warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
time_mix_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, int stride,
                       const float* __restrict__ norm, float eps, float out_scale, T* __restrict__ out, int out_stride,
                       int n_tokens, int heads, int dim) {
    pdl_launch_dependents();
    pdl_wait();
    const long long item = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads), head = (int)(item - (long long)t * heads);
    const float* row = o + (size_t)t * stride + (size_t)head * dim;
    const float* g = gate + (size_t)t * stride + (size_t)head * dim;
    float squares = 0.0f;
    for (int d = lane; d < dim; d += 32) squares = fmaf(row[d], row[d], squares);
    const float factor = out_scale / sqrtf(warp_sum(squares) / (float)dim + eps);
    for (int d = lane; d < dim; d += 32) {
        const float z = g[d];
        out[(size_t)t * out_stride + (size_t)head * dim + d] =
            from_float<T>(row[d] * factor * norm[(size_t)head * dim + d] * (z / (1.0f + expf(-z))));
    }
    if (head == heads - 1)                              // columns that pad the row to whole 16 bytes
        for (int d = heads * dim + lane; d < out_stride; d += 32) out[(size_t)t * out_stride + d] = from_float<T>(0.0f);
}

}  // namespace skv

using namespace skv;

static TimeMixBatch time_mix_batch(const int* positions, const int* token_seq, const int* cu_q, const int* slot_ids,
                                   float* state, long long state_stride, long long state_offset) {
    TimeMixBatch batch;
    batch.positions = positions; batch.token_seq = token_seq; batch.cu_q = cu_q; batch.slot_ids = slot_ids;
    batch.state = state; batch.state_stride = state_stride; batch.state_offset = state_offset;
    return batch;
}

// Floats of state a sequence needs: S twice and the mixer's last input twice.
SKV_EXPORT long long skv_time_mix_state_floats(int hidden, int heads, int dim) {
    return 2LL * heads * dim * dim + 2LL * hidden;
}

// h [n, hidden] and mixes [n_mixes, n, hidden] in the compute dtype, mu float [n_mixes, hidden].
SKV_EXPORT int skv_token_shift_mix(const void* h, const float* mu, void* mixes, int n, int hidden, int n_mixes, int heads,
                                   int dim, const int* positions, const int* token_seq, const int* cu_q,
                                   const int* slot_ids, float* state, long long state_stride, long long state_offset,
                                   cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hidden <= 0 || n_mixes <= 0 || n_mixes > TM_MAX_MIXES) return fail("skv_token_shift_mix", "1 to 8 mixes are served");
    if (!h || !mu || !mixes || !state) return fail("skv_token_shift_mix", "rows, factors, state and a place for the mixes are needed");
    const long long before_offset = 2LL * heads * dim * dim;
    const TimeMixBatch batch = time_mix_batch(positions, token_seq, cu_q, slot_ids, state, state_stride, state_offset);
    // eight channels a thread where every row that is read or written starts on 16 bytes (32 for floats)
    const bool vec = hidden % 8 == 0 && !(((uintptr_t)h | (uintptr_t)mixes | (uintptr_t)mu | (uintptr_t)state) & 31) &&
                     state_stride % 8 == 0 && (state_offset + before_offset) % 8 == 0;
    if (vec)
        return launch_pdl("skv_token_shift_mix", token_shift_mix_kernel<skv_t, true>, dim3(n), dim3(256), 0, stream,
                          (const skv_t*)h, mu, (skv_t*)mixes, n, hidden, n_mixes, before_offset, batch);
    return launch_pdl("skv_token_shift_mix", token_shift_mix_kernel<skv_t, false>, dim3(n), dim3(256), 0, stream,
                      (const skv_t*)h, mu, (skv_t*)mixes, n, hidden, n_mixes, before_offset, batch);
}

// lora float [n, lora_stride] (the first `rank` columns count), w2t [rank, channels] (the weight transposed) in the
// compute dtype.
SKV_EXPORT int skv_time_mix_decay(const float* lora, int lora_stride, int rank, const void* w2, const float* w0,
                                  float* decay, int n, int channels, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (rank <= 0 || rank > 8192 || channels <= 0 || lora_stride < rank) return fail("skv_time_mix_decay", "sizes do not agree");
    if (!lora || !w2 || !w0 || !decay) return fail("skv_time_mix_decay", "a pointer is missing");
    if ((size_t)TM_DECAY_TOKENS * rank * sizeof(float) > 48 * 1024) return fail("skv_time_mix_decay", "the rank is too large");
    return launch_pdl("skv_time_mix_decay", time_mix_decay_kernel<skv_t>,
                      dim3((n + TM_DECAY_TOKENS - 1) / TM_DECAY_TOKENS, (channels + 255) / 256), dim3(256), (size_t)TM_DECAY_TOKENS * rank * sizeof(float), stream, lora, lora_stride, rank,
                      (const skv_t*)w2, w0, decay, n, channels);
}

// r, k, v, decay, out: float [n, stride] with head `a` at columns a * dim; bonus float [heads, dim]; h [n, hidden] in the
// compute dtype.
SKV_EXPORT int skv_time_mix_scan(const float* r, const float* k, const float* v, const float* decay, int stride,
                                 const float* bonus, float* out, const void* h, int hidden, int n_seqs, int heads, int dim,
                                 const int* positions, const int* token_seq, const int* cu_q, const int* slot_ids,
                                 float* state, long long state_stride, long long state_offset, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (heads <= 0 || dim <= 0 || dim > 32 * TM_REGS || heads > 65535)
        return fail("skv_time_mix_scan", "heads of 1 to 512 numbers are served");
    if (!r || !k || !v || !decay || !bonus || !out || !h || !state) return fail("skv_time_mix_scan", "a pointer is missing");
    // Few blocks (one prompt alone): four key channels a thread, so that a head's work spreads over four times the
    // threads; else sixteen.
    const long long blocks = (long long)n_seqs * heads;
    const int regs = blocks * 4 <= sm_count() * 2 && dim <= 128 ? 4 : TM_REGS;
    int key_split = 1;
    while (key_split * regs < dim) key_split *= 2;
    // The value columns of a head are cut into slices (blocks) so that a step of few sequences still fills the GPU: a
    // slice of at least 8 columns, a multiple of 4 (the staged rows stay 16-byte aligned), at most 256 threads.
    int cols = min((dim + 3) & ~3, 256 / key_split);
    if (blocks < sm_count()) {
        const int wanted = (int)((sm_count() + blocks - 1) / blocks);
        const int fewer = (((dim + wanted - 1) / wanted) + 3) & ~3;
        cols = max(8, min(cols, fewer));
    }
    const int slices = (dim + cols - 1) / cols;
    const int padded = key_split * (regs == 16 ? TimeMixLayout<16>::stride : TimeMixLayout<4>::stride);
    int chunk = (int)(20 * 1024 / ((3 * (size_t)padded + cols) * sizeof(float)));       // two sets within 40 KB
    chunk = chunk < 1 ? 1 : (chunk > 16 ? 16 : chunk);
    const size_t smem = 2 * (size_t)chunk * (3 * (size_t)padded + cols) * sizeof(float);
    const int threads = ((cols * key_split + 31) / 32) * 32;
    const TimeMixBatch batch = time_mix_batch(positions, token_seq, cu_q, slot_ids, state, state_stride, state_offset);
    if (regs == 4)
        return launch_pdl("skv_time_mix_scan", time_mix_scan_kernel<skv_t, 4>, dim3(n_seqs, heads, slices), dim3(threads), smem,
                          stream, r, k, v, decay, stride, bonus, out, (const skv_t*)h, hidden, heads, dim, key_split, cols,
                          chunk, batch);
    return launch_pdl("skv_time_mix_scan", time_mix_scan_kernel<skv_t, 16>, dim3(n_seqs, heads, slices), dim3(threads), smem,
                      stream, r, k, v, decay, stride, bonus, out, (const skv_t*)h, hidden, heads, dim, key_split, cols,
                      chunk, batch);
}

// o and gate float [n, stride]; norm float [heads * dim]; out [n, out_stride] in the compute dtype.
SKV_EXPORT int skv_time_mix_finish(const float* o, const float* gate, int stride, const float* norm, float eps,
                                   float out_scale, void* out, int out_stride, int n, int heads, int dim,
                                   cudaStream_t stream) {
    if (n <= 0) return 0;
    if (heads <= 0 || dim <= 0 || out_stride < heads * dim) return fail("skv_time_mix_finish", "sizes do not agree");
    if (!o || !gate || !norm || !out) return fail("skv_time_mix_finish", "a pointer is missing");
    const long long items = (long long)n * heads;
    return launch_pdl("skv_time_mix_finish", time_mix_finish_kernel<skv_t>, dim3((unsigned)((items + 7) / 8)), dim3(256), 0,
                      stream, o, gate, stride, norm, eps, out_scale, (skv_t*)out, out_stride, n, heads, dim);
}
