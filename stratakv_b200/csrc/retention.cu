// Retention: linear attention with a fixed decay per head, over packed steps of several sequences.
//
// A float row of the layer's fused projection holds q [H][d], k [H][d], v [H][dv] and the gate g [H][dv].  Per head,
// with a = decay[head] and position p of a sequence:
//
//   q_p, k_p  rotated (first `rotated` numbers, number i with number i + rotated/2), k_p then times d^-1/2
//   S_p = a S_(p-1) + k_p v_p^T          (d x dv, zero before the first token)
//   o_p = S_p^T q_p;   out_p = o_p / sqrt(mean(o_p^2) + eps) * silu(g_p)        (compute dtype, input of Wo)
//
// Everything here is float.  Per sequence the cache keeps S twice, one row per slot [2][H][d][dv]: a step reads the
// half of the position before its first (by that position's parity) and writes the half of its last, so a one-token
// step that runs twice (a graph's capture after its warm-up) computes the same thing both times.
//
// One token a sequence: one kernel, a block per (head, sequence), does all of it.  Longer steps: queries and keys are
// rotated in place, then the sequence's tokens are cut into chunks of 32.  With S the state before a chunk of L tokens,
//   o_i    = a^(i+1) S^T q_i + sum_(j<=i) a^(i-j) (q_i . k_j) v_j             (i, j count within the chunk)
//   S_next = a^L S + sum_j a^(L-1-j) k_j v_j^T
// so a first kernel leaves every chunk's own sum (the second term of S_next), a second walks the chunks of a sequence
// and replaces each sum by the state before its chunk, and a third makes the outputs of all chunks side by side.
#include "common.cuh"

namespace skv {

constexpr int RET_CHUNK = 32;
constexpr int RET_THREADS = 256;
constexpr int RET_WARPS = RET_THREADS / 32;

struct RetentionBatch {
    const int* positions;      // [tokens]
    const int* token_seq;      // [tokens]
    const int* cu_q;           // [seqs + 1]
    const int* slot_ids;       // [seqs]
    float* state;              // [slots][state_stride]
    int state_stride;          // floats per slot: at least 2 * H * d * dv
};

struct RetentionShape {
    int heads, dim, vdim;
    int row_stride;            // floats per row of the fused projection
    int rotated, table_len;    // the rotation: how many numbers of a head turn, and the table's positions
};

// a^n for a decay 0 <= a <= 1 and a small whole n, in float: exp(n ln a).
__device__ __forceinline__ float decay_power(float log_decay, float decay, int n) {
    if (n == 0) return 1.0f;
    if (decay <= 0.0f) return 0.0f;
    return expf((float)n * log_decay);
}

__device__ __forceinline__ float rotated_value(const float* x, int j, int rotated, const float* cos_sin) {
    if (j >= rotated) return x[j];
    const int half = rotated >> 1;
    if (j < half) return x[j] * cos_sin[2 * j] - x[j + half] * cos_sin[2 * j + 1];
    const int i = j - half;
    return x[j] * cos_sin[2 * i] + x[i] * cos_sin[2 * i + 1];
}

// ---- one token a sequence ----------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(RET_THREADS)
retention_decode_kernel(const float* __restrict__ fused, const float* __restrict__ rotation,
                        const float* __restrict__ decay, float eps, T* __restrict__ out, int out_stride,
                        const RetentionShape shape, const RetentionBatch batch) {
    extern __shared__ __align__(16) float ret_smem[];
    const int H = shape.heads, d = shape.dim, dv = shape.vdim;
    float* q = ret_smem;                      // [d]
    float* k = q + d;                         // [d]
    float* v = k + d;                         // [dv]
    float* partial = v + dv;                  // [RET_WARPS][dv]
    __shared__ float reduce[33];
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, s = blockIdx.y;
    const int t = batch.cu_q[s];
    const int p = batch.positions[t];
    const float* row = fused + (size_t)t * shape.row_stride;
    const float* cos_sin = rotation ? rotation + (size_t)min(p, shape.table_len - 1) * shape.rotated : nullptr;
    const int turn = rotation ? shape.rotated : 0;
    const float key_scale = 1.0f / sqrtf((float)d);
    for (int j = threadIdx.x; j < d; j += RET_THREADS) {
        q[j] = rotated_value(row + (size_t)head * d, j, turn, cos_sin);
        k[j] = rotated_value(row + (size_t)(H + head) * d, j, turn, cos_sin) * key_scale;
    }
    for (int e = threadIdx.x; e < dv; e += RET_THREADS) v[e] = row[(size_t)2 * H * d + (size_t)head * dv + e];
    __syncthreads();
    const size_t half_size = (size_t)H * d * dv;
    float* slot = batch.state + (size_t)batch.slot_ids[s] * batch.state_stride;
    const float* before = p > 0 ? slot + (size_t)((p - 1) & 1) * half_size + (size_t)head * d * dv : nullptr;
    float* after = slot + (size_t)(p & 1) * half_size + (size_t)head * d * dv;
    const float a = decay[head];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e0 = 0; e0 < dv; e0 += 32) {
        const int e = e0 + lane;
        float acc = 0.0f;
        if (e < dv) {
            const float ve = v[e];
            for (int j = warp; j < d; j += RET_WARPS) {
                const size_t at = (size_t)j * dv + e;
                const float fresh = fmaf(a, before ? before[at] : 0.0f, k[j] * ve);
                after[at] = fresh;
                acc = fmaf(fresh, q[j], acc);
            }
            partial[warp * dv + e] = acc;
        }
    }
    __syncthreads();
    float squares = 0.0f;
    for (int e = threadIdx.x; e < dv; e += RET_THREADS) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < RET_WARPS; ++w) o += partial[w * dv + e];
        v[e] = o;                              // (each thread replaces the values it alone reads from here on)
        squares = fmaf(o, o, squares);
    }
    const float factor = 1.0f / sqrtf(block_sum(squares, reduce) / (float)dv + eps);
    const float* gate = row + (size_t)2 * H * d + (size_t)H * dv + (size_t)head * dv;
    T* out_row = out + (size_t)t * out_stride + (size_t)head * dv;
    for (int e = threadIdx.x; e < dv; e += RET_THREADS) {
        const float g = gate[e];
        out_row[e] = from_float<T>(v[e] * factor * (g / (1.0f + expf(-g))));
    }
    if (head == H - 1)
        for (int c = H * dv + threadIdx.x; c < out_stride; c += RET_THREADS) out[(size_t)t * out_stride + c] = from_float<T>(0.0f);
}

// ---- longer steps ----------------------------------------------------------------------------------------------
// Queries and keys of every token rotated in place; keys also times d^-1/2.
__global__ void __launch_bounds__(RET_THREADS)
retention_rotate_kernel(float* __restrict__ fused, const float* __restrict__ rotation, int n_tokens,
                        const RetentionShape shape, const int* __restrict__ positions) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int H = shape.heads, d = shape.dim;
    const int turn = rotation ? shape.rotated : 0, half = turn >> 1;
    const float* cos_sin = rotation ? rotation + (size_t)min(positions[t], shape.table_len - 1) * shape.rotated : nullptr;
    const float key_scale = 1.0f / sqrtf((float)d);
    float* row = fused + (size_t)t * shape.row_stride;
    for (int idx = threadIdx.x; idx < H * d; idx += RET_THREADS) {
        const int head = idx / d, j = idx - head * d;
        float* qh = row + (size_t)head * d;
        float* kh = row + (size_t)(H + head) * d;
        if (j < half) {                        // this thread turns the pair (j, j + half) of the query and of the key
            const float c = cos_sin[2 * j], sn = cos_sin[2 * j + 1];
            const float qu = qh[j], qv = qh[j + half], ku = kh[j], kv = kh[j + half];
            qh[j] = qu * c - qv * sn;
            qh[j + half] = qv * c + qu * sn;
            kh[j] = (ku * c - kv * sn) * key_scale;
            kh[j + half] = (kv * c + ku * sn) * key_scale;
        } else if (j >= turn) {
            kh[j] *= key_scale;
        }
    }
}

// sums [seqs][max_chunks][H][d][dv]: chunk c of sequence s gets sum_j a^(L-1-j) k_j v_j^T.
__global__ void __launch_bounds__(RET_THREADS)
retention_chunk_sum_kernel(const float* __restrict__ fused, const float* __restrict__ decay, float* __restrict__ sums,
                           int max_chunks, const RetentionShape shape, const int* __restrict__ cu_q) {
    extern __shared__ __align__(16) float ret_smem[];
    const int H = shape.heads, d = shape.dim, dv = shape.vdim;
    float* ks = ret_smem;                     // [RET_CHUNK][d], already weighed by the decay
    float* vs = ks + RET_CHUNK * d;           // [RET_CHUNK][dv]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, head = blockIdx.y, s = blockIdx.z;
    const int first = cu_q[s] + c * RET_CHUNK, L = min(RET_CHUNK, cu_q[s + 1] - first);
    if (L <= 0) return;
    const float a = decay[head], log_a = a > 0.0f ? logf(a) : 0.0f;
    for (int idx = threadIdx.x; idx < L * d; idx += RET_THREADS) {
        const int j = idx / d, col = idx - j * d;
        ks[idx] = fused[(size_t)(first + j) * shape.row_stride + (size_t)(H + head) * d + col] * decay_power(log_a, a, L - 1 - j);
    }
    for (int idx = threadIdx.x; idx < L * dv; idx += RET_THREADS) {
        const int j = idx / dv, col = idx - j * dv;
        vs[idx] = fused[(size_t)(first + j) * shape.row_stride + (size_t)2 * H * d + (size_t)head * dv + col];
    }
    __syncthreads();
    float* mine = sums + (((size_t)s * max_chunks + c) * H + head) * (size_t)d * dv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a tile of 64 rows (8 per warp) by 128 columns (4 per lane) at a time
    for (int r0 = 0; r0 < d; r0 += 64)
        for (int e0 = 0; e0 < dv; e0 += 128) {
            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) acc[i][jj] = 0.0f;
            for (int j = 0; j < L; ++j) {
                float kr[8], vc[4];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = r0 + warp + RET_WARPS * i;
                    kr[i] = r < d ? ks[j * d + r] : 0.0f;
                }
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int e = e0 + lane + 32 * jj;
                    vc[jj] = e < dv ? vs[j * dv + e] : 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) acc[i][jj] = fmaf(kr[i], vc[jj], acc[i][jj]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = r0 + warp + RET_WARPS * i;
                if (r >= d) continue;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int e = e0 + lane + 32 * jj;
                    if (e < dv) mine[(size_t)r * dv + e] = acc[i][jj];
                }
            }
        }
}

// Walks a sequence's chunks: every chunk's sum is replaced by the state before the chunk; the state after the last
// chunk goes to the cache.
__global__ void __launch_bounds__(RET_THREADS)
retention_carry_kernel(const float* __restrict__ decay, float* __restrict__ sums, int max_chunks,
                       const RetentionShape shape, const RetentionBatch batch) {
    pdl_launch_dependents();
    pdl_wait();
    const int H = shape.heads, d = shape.dim, dv = shape.vdim;
    const int head = blockIdx.y, s = blockIdx.z;
    const int at = blockIdx.x * RET_THREADS + threadIdx.x;
    if (at >= d * dv) return;
    const int first = batch.cu_q[s], count = batch.cu_q[s + 1] - first;
    if (count <= 0) return;
    const int p_first = batch.positions[first], p_last = p_first + count - 1;
    const size_t half_size = (size_t)H * d * dv, mine = (size_t)head * d * dv + at;
    float* slot = batch.state + (size_t)batch.slot_ids[s] * batch.state_stride;
    float S = p_first > 0 ? slot[(size_t)((p_first - 1) & 1) * half_size + mine] : 0.0f;
    const float a = decay[head], log_a = a > 0.0f ? logf(a) : 0.0f;
    const int chunks = (count + RET_CHUNK - 1) / RET_CHUNK;
    const float whole = decay_power(log_a, a, RET_CHUNK);              // the decay over a full chunk
    const size_t stride = (size_t)H * d * dv;                          // from a chunk's cell to the next chunk's
    float* cells = sums + ((size_t)s * max_chunks * H) * (size_t)d * dv + mine;
    // eight chunks' sums are fetched before any state is stored over them: a store between two loads of the same
    // array would make each load wait for the one before, and the walk would take a memory latency per chunk
    constexpr int AHEAD = 8;
    for (int c0 = 0; c0 < chunks; c0 += AHEAD) {
        float own[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) own[i] = c0 + i < chunks ? __ldcg(cells + (size_t)(c0 + i) * stride) : 0.0f;
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            const int c = c0 + i;
            if (c < chunks) {
                cells[(size_t)c * stride] = S;
                const int L = min(RET_CHUNK, count - c * RET_CHUNK);
                S = fmaf(L == RET_CHUNK ? whole : decay_power(log_a, a, L), S, own[i]);
            }
        }
    }
    slot[(size_t)(p_last & 1) * half_size + mine] = S;
}

// The outputs of one chunk of one head: before [d][dv] is the state before the chunk (what retention_carry_kernel left).
template <typename T>
__global__ void __launch_bounds__(RET_THREADS)
retention_chunk_output_kernel(const float* __restrict__ fused, const float* __restrict__ decay,
                              const float* __restrict__ sums, int max_chunks, float eps, T* __restrict__ out,
                              int out_stride, const RetentionShape shape, const int* __restrict__ cu_q) {
    extern __shared__ __align__(16) float ret_smem[];
    const int H = shape.heads, d = shape.dim, dv = shape.vdim;
    const int ld = d + 1;                                 // rows of q and k one float apart from a multiple of the banks
    float* qs = ret_smem;                                 // [RET_CHUNK][ld]
    float* ks = qs + RET_CHUNK * ld;                      // [RET_CHUNK][ld]
    float* vs = ks + RET_CHUNK * ld;                      // [RET_CHUNK][dv]
    float* weights = vs + RET_CHUNK * dv;                 // [RET_CHUNK][RET_CHUNK + 1]: a^(i-j) (q_i . k_j), j <= i
    float* os = weights + RET_CHUNK * (RET_CHUNK + 1);    // [RET_CHUNK][dv]
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x, head = blockIdx.y, s = blockIdx.z;
    const int first = cu_q[s] + c * RET_CHUNK, L = min(RET_CHUNK, cu_q[s + 1] - first);
    if (L <= 0) return;
    const float a = decay[head], log_a = a > 0.0f ? logf(a) : 0.0f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int idx = threadIdx.x; idx < RET_CHUNK * d; idx += RET_THREADS) {
        const int j = idx / d, col = idx - j * d;
        const float* row = fused + (size_t)(first + j) * shape.row_stride;
        qs[j * ld + col] = j < L ? row[(size_t)head * d + col] : 0.0f;
        ks[j * ld + col] = j < L ? row[(size_t)(H + head) * d + col] : 0.0f;
    }
    for (int idx = threadIdx.x; idx < RET_CHUNK * dv; idx += RET_THREADS) {
        const int j = idx / dv, col = idx - j * dv;
        vs[idx] = j < L ? fused[(size_t)(first + j) * shape.row_stride + (size_t)2 * H * d + (size_t)head * dv + col] : 0.0f;
    }
    __syncthreads();
    // weights: row i = warp + 8 ii, column j = lane
    {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int col = 0; col < d; ++col) {
            const float kj = ks[lane * ld + col];
#pragma unroll
            for (int ii = 0; ii < 4; ++ii) acc[ii] = fmaf(qs[(warp + RET_WARPS * ii) * ld + col], kj, acc[ii]);
        }
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
            const int i = warp + RET_WARPS * ii, j = lane;
            weights[i * (RET_CHUNK + 1) + j] = j <= i ? acc[ii] * decay_power(log_a, a, i - j) : 0.0f;
        }
    }
    __syncthreads();
    const float* before = sums + (((size_t)s * max_chunks + c) * H + head) * (size_t)d * dv;
    float carry[4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) carry[ii] = decay_power(log_a, a, warp + RET_WARPS * ii + 1);
    // outputs: rows i = warp + 8 ii, columns e = e0 + lane + 32 jj
    for (int e0 = 0; e0 < dv; e0 += 128) {
        float acc[4][4];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = 0.0f;
        for (int col = 0; col < d; ++col) {               // what the state before the chunk gives
            float sv[4];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int e = e0 + lane + 32 * jj;
                sv[jj] = e < dv ? before[(size_t)col * dv + e] : 0.0f;
            }
#pragma unroll
            for (int ii = 0; ii < 4; ++ii) {
                const float qi = qs[(warp + RET_WARPS * ii) * ld + col];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = fmaf(qi, sv[jj], acc[ii][jj]);
            }
        }
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) acc[ii][jj] *= carry[ii];
        for (int j = 0; j < L; ++j) {                     // what the chunk's own tokens give
            float vv[4];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int e = e0 + lane + 32 * jj;
                vv[jj] = e < dv ? vs[j * dv + e] : 0.0f;
            }
#pragma unroll
            for (int ii = 0; ii < 4; ++ii) {
                const float w = weights[(warp + RET_WARPS * ii) * (RET_CHUNK + 1) + j];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = fmaf(w, vv[jj], acc[ii][jj]);
            }
        }
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int e = e0 + lane + 32 * jj;
                if (e < dv) os[(warp + RET_WARPS * ii) * dv + e] = acc[ii][jj];
            }
    }
    __syncwarp();                                         // (a warp reads back only the rows it wrote itself)
    // every head's output divided by its root mean square, times silu(gate): a warp takes its own four rows
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
        const int i = warp + RET_WARPS * ii;
        if (i >= L) continue;
        float squares = 0.0f;
        for (int e = lane; e < dv; e += 32) squares = fmaf(os[i * dv + e], os[i * dv + e], squares);
        const float factor = 1.0f / sqrtf(warp_sum(squares) / (float)dv + eps);
        const size_t t = (size_t)first + i;
        const float* gate = fused + t * shape.row_stride + (size_t)2 * H * d + (size_t)H * dv + (size_t)head * dv;
        T* out_row = out + t * out_stride + (size_t)head * dv;
        for (int e = lane; e < dv; e += 32) {
            const float g = gate[e];
            out_row[e] = from_float<T>(os[i * dv + e] * factor * (g / (1.0f + expf(-g))));
        }
        if (head == H - 1)
            for (int col = H * dv + lane; col < out_stride; col += 32) out[t * out_stride + col] = from_float<T>(0.0f);
    }
}

static int reserve_shared(const void* kernel, size_t bytes, const char* name) {
    if (bytes <= 48 * 1024) return 0;
    if (bytes > 200 * 1024) return fail(name, "the head sizes are too large for this kernel's shared memory");
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
        return fail(name, "cannot reserve shared memory");
    return 0;
}

}  // namespace skv

using namespace skv;

// Floats of scratch that skv_retention needs for a step whose longest sequence brings max_q_len tokens (0 for one
// token a sequence).
SKV_EXPORT long long skv_retention_scratch(int n_seqs, int max_q_len, int heads, int dim, int vdim) {
    if (max_q_len <= 1) return 0;
    return (long long)n_seqs * ((max_q_len + RET_CHUNK - 1) / RET_CHUNK) * heads * dim * vdim;
}

// fused: float [n_tokens, row_stride], rows [q | k | v | gate]; queries and keys are rotated in place where a step
// brings more than one token a sequence.  rotation: float [table_len][rotated / 2][2] or null.  decay: float [heads].
// out: [n_tokens, out_stride] in the compute dtype.  state: float [slots][state_stride].
SKV_EXPORT int skv_retention(float* fused, int row_stride, const float* rotation, int rotated, int table_len,
                             const float* decay, float eps, void* out, int out_stride, float* scratch, int n_tokens,
                             int n_seqs, int heads, int dim, int vdim, int max_q_len, const int* positions,
                             const int* token_seq, const int* cu_q, const int* slot_ids, float* state, int state_stride,
                             cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (!fused || !decay || !out || !positions || !cu_q || !slot_ids || !state)
        return fail("skv_retention", "the projection's rows, the decays, the step's metadata and the state are needed");
    if (heads <= 0 || dim <= 0 || vdim <= 0 || max_q_len <= 0) return fail("skv_retention", "sizes must be positive");
    if (heads > 65535 || n_seqs > 65535) return fail("skv_retention", "too many heads or sequences in one step");
    if (row_stride < 2 * heads * (dim + vdim)) return fail("skv_retention", "a row is shorter than its queries, keys, values and gates");
    if (out_stride < heads * vdim) return fail("skv_retention", "a row of the output is shorter than its heads");
    if ((long long)state_stride < 2LL * heads * dim * vdim) return fail("skv_retention", "a slot's state is too small: 2 * heads * dim * vdim floats are needed");
    if (rotation && (rotated <= 0 || rotated % 2 || rotated > dim || table_len <= 0))
        return fail("skv_retention", "the rotated numbers must be an even count within a head");
    const RetentionShape shape = {heads, dim, vdim, row_stride, rotation ? rotated : 0, table_len};
    const RetentionBatch batch = {positions, token_seq, cu_q, slot_ids, state, state_stride};
    if (max_q_len == 1) {
        if (n_tokens != n_seqs) return fail("skv_retention", "one token a sequence means as many tokens as sequences");
        const size_t smem = (size_t)(2 * dim + vdim + RET_WARPS * vdim) * sizeof(float);
        auto kernel = retention_decode_kernel<skv_t>;
        if (int code = reserve_shared((const void*)kernel, smem, "skv_retention")) return code;
        return launch_pdl("skv_retention", kernel, dim3(heads, n_seqs), dim3(RET_THREADS), smem, stream,
                          (const float*)fused, rotation, decay, eps, (skv_t*)out, out_stride, shape, batch);
    }
    if (!scratch) return fail("skv_retention", "a step of more than one token a sequence needs scratch for its chunks");
    const int max_chunks = (max_q_len + RET_CHUNK - 1) / RET_CHUNK;
    if (max_chunks > 0x7fffffff / 2) return fail("skv_retention", "too many tokens of one sequence in one step");
    if (int code = launch_pdl("skv_retention", retention_rotate_kernel, dim3(n_tokens), dim3(RET_THREADS), 0, stream,
                              fused, rotation, n_tokens, shape, positions))
        return code;
    const size_t sum_smem = (size_t)RET_CHUNK * (dim + vdim) * sizeof(float);
    if (int code = reserve_shared((const void*)retention_chunk_sum_kernel, sum_smem, "skv_retention")) return code;
    if (int code = launch_pdl("skv_retention", retention_chunk_sum_kernel, dim3(max_chunks, heads, n_seqs),
                              dim3(RET_THREADS), sum_smem, stream, (const float*)fused, decay, scratch, max_chunks, shape, cu_q))
        return code;
    if (int code = launch_pdl("skv_retention", retention_carry_kernel,
                              dim3((dim * vdim + RET_THREADS - 1) / RET_THREADS, heads, n_seqs), dim3(RET_THREADS), 0,
                              stream, decay, scratch, max_chunks, shape, batch))
        return code;
    const size_t out_smem = (size_t)(2 * RET_CHUNK * (dim + 1) + 2 * RET_CHUNK * vdim + RET_CHUNK * (RET_CHUNK + 1)) * sizeof(float);
    auto kernel = retention_chunk_output_kernel<skv_t>;
    if (int code = reserve_shared((const void*)kernel, out_smem, "skv_retention")) return code;
    return launch_pdl("skv_retention", kernel, dim3(max_chunks, heads, n_seqs), dim3(RET_THREADS), out_smem, stream,
                      (const float*)fused, decay, (const float*)scratch, max_chunks, eps, (skv_t*)out, out_stride, shape, cu_q);
}
