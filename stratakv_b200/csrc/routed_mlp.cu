// A routed feed-forward (mixture of experts): router, sort of the (token, choice) pairs by expert, projections over
// the sorted pairs with each expert's own weights, and the weighted sum.
//
//   s = sigmoid(router . h)                     float sums, one score per expert (or softmax over all experts)
//   chosen: the `top` largest s + correction    (the lower index among equals; the correction chooses only); with
//                                               groups: the experts form equal groups of neighbours, a group scores
//                                               what its best expert does, and only the `keep` best groups' experts
//                                               can be chosen
//   weight of a chosen expert: s * scale        (renormalize: s divided by the chosen scores' sum + renorm_eps first)
//   share = sigmoid(shared_gate . h)            one number per token for a shared expert, if the layer has one
//
// Nothing is read back to the host: the number of pairs of every expert stays on the device (offsets [experts + 1]),
// and the projections are launched over an upper bound of row tiles, each of which looks up its expert.
#include "common.cuh"

namespace skv {

constexpr int ROUTE_THREADS = 256;
constexpr int ROUTE_MAX_EXPERTS = 1024;
constexpr int ROUTE_MAX_TOP = 16;

// ---- router ------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_tokens_kernel(const T* __restrict__ h, const T* __restrict__ router, const float* __restrict__ correction,
                    const T* __restrict__ shared_gate, int hidden, int experts, int top, float scale, int renormalize,
                    int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ share, int softmax,
                    int groups, int keep, float renorm_eps) {
    extern __shared__ __align__(16) float route_smem[];
    float* row = route_smem;                  // [hidden]
    float* score = row + hidden;              // [experts]
    float* choice = score + experts;          // [experts]
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int w = threadIdx.x; w < hidden; w += ROUTE_THREADS) row[w] = to_float(h[(size_t)t * hidden + w]);
    __syncthreads();
    const int dots = experts + (shared_gate ? 1 : 0);
    for (int e = warp; e < dots; e += ROUTE_THREADS / 32) {
        const T* w_row = e < experts ? router + (size_t)e * hidden : shared_gate;
        float acc = 0.0f;
        for (int w = lane; w < hidden; w += 32) acc = fmaf(to_float(w_row[w]), row[w], acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            const float s = softmax && e < experts ? acc : 1.0f / (1.0f + expf(-acc));
            if (e < experts) {
                score[e] = s;
                choice[e] = correction ? s + correction[e] : s;
            } else {
                share[t] = s;
            }
        }
    }
    __syncthreads();
    if (warp != 0) return;
    if (softmax) {
        // the logits become exp(z - max) / sum over all experts
        float top_logit = -INFINITY;
        for (int e = lane; e < experts; e += 32) top_logit = fmaxf(top_logit, score[e]);
        top_logit = warp_max(top_logit);
        float total = 0.0f;
        for (int e = lane; e < experts; e += 32) {
            const float w = expf(score[e] - top_logit);
            score[e] = w;
            total += w;
        }
        total = warp_sum(total);
        __syncwarp();
        for (int e = lane; e < experts; e += 32) {
            const float s = score[e] / total;
            score[e] = s;
            choice[e] = correction ? s + correction[e] : s;
        }
        __syncwarp();
    }
    if (groups > 1) {
        // `keep` rounds: the group whose best expert scores most (the lower index among equals) is kept, which an
        // infinity in its members' places says; the members of all other groups then leave the choice
        const int size = experts / groups;
        for (int round = 0; round < keep; ++round) {
            float best = 0.0f;
            int best_at = -1;
            for (int g = lane; g < groups; g += 32) {
                bool taken = false;
                for (int e = 0; e < size; ++e) taken = taken || choice[g * size + e] == INFINITY;
                if (taken) continue;
                float top_score = choice[g * size];
                for (int e = 1; e < size; ++e) top_score = fmaxf(top_score, choice[g * size + e]);
                if (best_at < 0 || top_score > best) {
                    best = top_score;
                    best_at = g;
                }
            }
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) {
                const float other = __shfl_xor_sync(0xffffffffu, best, offset);
                const int other_at = __shfl_xor_sync(0xffffffffu, best_at, offset);
                if (other_at >= 0 && (best_at < 0 || other > best || (other == best && other_at < best_at))) {
                    best = other;
                    best_at = other_at;
                }
            }
            __syncwarp();
            if (best_at >= 0)
                for (int e = lane; e < size; e += 32) choice[best_at * size + e] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32) {
            const float c = choice[e];
            const float s = score[e];
            choice[e] = c == INFINITY ? (correction ? s + correction[e] : s) : __int_as_float(0x7fc00000);
        }
        __syncwarp();
    }
    // `top` rounds: the largest choice score left (the lower index among equals); an expert that has been taken is
    // marked with a value that is not a number, which the search passes over
    float picked_sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = 0.0f;
        int best_at = -1;
        for (int e = lane; e < experts; e += 32) {
            const float c = choice[e];
            if (c != c) continue;
            if (best_at < 0 || c > best) {
                best = c;
                best_at = e;
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, best, offset);
            const int other_at = __shfl_xor_sync(0xffffffffu, best_at, offset);
            if (other_at >= 0 && (best_at < 0 || other > best || (other == best && other_at < best_at))) {
                best = other;
                best_at = other_at;
            }
        }
        if (best_at < 0) best_at = k;                 // (only where the scores are not numbers)
        const float s = score[best_at];
        picked_sum += s;
        __syncwarp();
        if (lane == 0) {
            chosen[(size_t)t * top + k] = best_at;
            weights[(size_t)t * top + k] = s;
            choice[best_at] = __int_as_float(0x7fc00000);
        }
        __syncwarp();
    }
    if (lane < top) {
        float w = weights[(size_t)t * top + lane];
        if (renormalize) w = w / (picked_sum + renorm_eps);
        weights[(size_t)t * top + lane] = w * scale;
    }
}

// ---- counting sort of the pairs by expert ----------------------------------------------------------------------------
// One block.  offsets [experts + 1]; order[p] = token of sorted pair p; place[pair] = where the pair went.
__global__ void __launch_bounds__(1024)
sort_by_expert_kernel(const int* __restrict__ chosen, int pairs, int top, int experts, int* __restrict__ offsets,
                      int* __restrict__ order, int* __restrict__ place) {
    __shared__ int counts[ROUTE_MAX_EXPERTS];
    __shared__ int cursor[ROUTE_MAX_EXPERTS];
    __shared__ int warp_totals[32];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    // exclusive scan of counts over up to 1024 experts: a thread per expert
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int mine = threadIdx.x < experts ? counts[threadIdx.x] : 0;
    int inclusive = mine;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const int below = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (lane >= offset) inclusive += below;
    }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
        int total = warp_totals[lane];
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
            const int below = __shfl_up_sync(0xffffffffu, total, offset);
            if (lane >= offset) total += below;
        }
        warp_totals[lane] = total;
    }
    __syncthreads();
    const int start = inclusive - mine + (warp > 0 ? warp_totals[warp - 1] : 0);
    if (threadIdx.x < experts) {
        cursor[threadIdx.x] = start;
        offsets[threadIdx.x] = start;
        if (threadIdx.x == experts - 1) offsets[experts] = start + mine;
    }
    __syncthreads();
    // Within an expert the pairs keep no particular order: every pair's result is computed from its own row alone,
    // so where it lies among its expert's rows changes nothing.
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < 0 || e >= experts) { place[p] = 0; continue; }
        const int at = atomicAdd(&cursor[e], 1);
        order[at] = p / top;
        place[p] = at;
    }
}

// ---- projections over the sorted pairs -----------------------------------------------------------------------------
constexpr int EXP_ROWS = 32, EXP_OUTS = 64, EXP_K = 32;

// Row tile `tile` of the launch: which expert, and which of its rows.  Tiles are counted expert by expert, each expert
// having ceil(rows / EXP_ROWS) of them; a tile beyond the last gets no expert.
__device__ __forceinline__ void find_tile(const int* __restrict__ offsets, int experts, int tile, int* expert, int* first,
                                          int* last) {
    int seen = 0;
    *expert = -1;
    for (int e = 0; e < experts; ++e) {
        const int lo = offsets[e], hi = offsets[e + 1];
        const int tiles = (hi - lo + EXP_ROWS - 1) / EXP_ROWS;
        if (tile < seen + tiles) {
            *expert = e;
            *first = lo + (tile - seen) * EXP_ROWS;
            *last = hi;
            return;
        }
        seen += tiles;
    }
}

// GATED: an expert's weight holds 2 N rows, in tiles of 16 (8 gate rows, then the 8 up rows that go with them, as the
// dense gated feed-forward packs them); out[., o] = act(gate_o . a) * (up_o . a).
template <typename TIn, typename TOut, bool GATED>
__global__ void __launch_bounds__(256)
expert_linear_kernel(const TIn* __restrict__ a, int a_stride, const int* __restrict__ rows, const TIn* __restrict__ w,
                     const int* __restrict__ offsets, TOut* __restrict__ out, int experts, int N, int K, int act) {
    __shared__ float as[EXP_ROWS][EXP_K + 1];
    __shared__ float ws[EXP_OUTS][EXP_K + 1];
    __shared__ float us[GATED ? EXP_OUTS : 1][EXP_K + 1];
    __shared__ int source[EXP_ROWS];
    __shared__ int tile_info[3];
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) find_tile(offsets, experts, blockIdx.y, &tile_info[0], &tile_info[1], &tile_info[2]);
    __syncthreads();
    const int expert = tile_info[0], first = tile_info[1], last = tile_info[2];
    if (expert < 0) return;
    const int count = min(EXP_ROWS, last - first);
    if (threadIdx.x < EXP_ROWS) {
        const int p = first + threadIdx.x;
        source[threadIdx.x] = threadIdx.x < count ? (rows ? rows[p] : p) : -1;
    }
    __syncthreads();
    const int o0 = blockIdx.x * EXP_OUTS;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const TIn* w_e = w + (size_t)expert * (GATED ? 2 : 1) * N * K;
    float acc[2][4] = {};
    float up[GATED ? 2 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += EXP_K) {
        for (int idx = threadIdx.x; idx < EXP_ROWS * EXP_K; idx += 256) {
            const int r = idx / EXP_K, k = idx % EXP_K;
            const int src = source[r];
            as[r][k] = src >= 0 && k0 + k < K ? to_float(a[(size_t)src * a_stride + k0 + k]) : 0.0f;
        }
        for (int idx = threadIdx.x; idx < EXP_OUTS * EXP_K; idx += 256) {
            const int r = idx / EXP_K, k = idx % EXP_K;
            const int o = o0 + r;
            if (GATED) {
                const size_t gate_row = (size_t)(o >> 3) * 16 + (o & 7);
                ws[r][k] = o < N && k0 + k < K ? to_float(w_e[gate_row * K + k0 + k]) : 0.0f;
                us[r][k] = o < N && k0 + k < K ? to_float(w_e[(gate_row + 8) * K + k0 + k]) : 0.0f;
            } else {
                ws[r][k] = o < N && k0 + k < K ? to_float(w_e[(size_t)o * K + k0 + k]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < EXP_K; ++k) {
            const float a0 = as[ty][k], a1 = as[ty + 16][k];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = ws[tx + 16 * j][k];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
                if (GATED) {
                    const float c = us[tx + 16 * j][k];
                    up[0][j] = fmaf(a0, c, up[0][j]);
                    up[1][j] = fmaf(a1, c, up[1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty + 16 * i;
        if (r >= count) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int o = o0 + tx + 16 * j;
            if (o >= N) continue;
            float v = acc[i][j];
            if (act == ACT_RELU2) v = relu_squared(v);
            else if (act == ACT_GELU_TANH) v = gelu_tanh(v);
            else if (act == ACT_SILU) v = v / (1.0f + expf(-v));
            if (GATED) v *= up[i][j];
            out[(size_t)(first + r) * N + o] = from_float<TOut>(v);
        }
    }
}

// ---- rows in sorted order --------------------------------------------------------------------------------------------
// out[p] = a[rows[p]] for every sorted pair p: the tensor-core projection reads whole tiles of neighbouring rows.
// Rows are K numbers, K * sizeof(T) a multiple of 16 bytes; a warp copies a row.
template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ a, int a_stride, const int* __restrict__ rows, T* __restrict__ out, int pairs, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int p = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (p >= pairs) return;
    const uint4* src = (const uint4*)(a + (size_t)rows[p] * a_stride);
    uint4* dst = (uint4*)(out + (size_t)p * K);
    const int pieces = K * (int)sizeof(T) / 16;
    for (int i = lane; i < pieces; i += 32) dst[i] = src[i];
}

// ---- the weighted sum ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
combine_experts_kernel(const float* __restrict__ results, const int* __restrict__ place, const float* __restrict__ weights,
                       const float* __restrict__ shared, const float* __restrict__ share, float* __restrict__ x,
                       int hidden, int top, int add) {
    __shared__ int where[ROUTE_MAX_TOP];
    __shared__ float weight[ROUTE_MAX_TOP];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (threadIdx.x < top) {
        where[threadIdx.x] = place[(size_t)t * top + threadIdx.x];
        weight[threadIdx.x] = weights[(size_t)t * top + threadIdx.x];
    }
    __syncthreads();
    const float gate = shared ? (share ? share[t] : 1.0f) : 0.0f;
    for (int w = threadIdx.x; w < hidden; w += 256) {
        float total = 0.0f;
        for (int k = 0; k < top; ++k) total = fmaf(weight[k], results[(size_t)where[k] * hidden + w], total);
        if (shared) total = fmaf(gate, shared[(size_t)t * hidden + w], total);
        const size_t at = (size_t)t * hidden + w;
        x[at] = add ? x[at] + total : total;
    }
}

#if SKV_DTYPE == SKV_BF16
// gemm_tcgen05.cu: the tensor-memory GEMM over rows sorted by group
int grouped_linear_tcgen05(const void* a, const void* w, const int* offsets, void* out, int out_is_float, int rows,
                           int groups, int N, int K, act_t act, int gated, int* flag, cudaStream_t stream);
#endif

}  // namespace skv

using namespace skv;

// h [n, hidden], router [experts, hidden], shared_gate [hidden] or null in the compute dtype; correction float
// [experts] or null.  chosen int [n, top], weights float [n, top], share float [n] (with shared_gate).
SKV_EXPORT int skv_route_tokens(const void* h, const void* router, const float* correction, const void* shared_gate,
                                int n, int hidden, int experts, int top, float scale, int renormalize, int* chosen,
                                float* weights, float* share, int softmax, int groups, int keep, float renorm_eps,
                                cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hidden <= 0 || experts <= 0 || experts > ROUTE_MAX_EXPERTS || top <= 0 || top > experts || top > ROUTE_MAX_TOP)
        return fail("skv_route_tokens", "1 to 16 of 1 to 1024 experts are served");
    if (!h || !router || !chosen || !weights || (shared_gate && !share))
        return fail("skv_route_tokens", "the rows, the router and places for the choice are needed");
    if (groups > 1 && (experts % groups != 0 || keep <= 0 || keep > groups || keep * (experts / groups) < top))
        return fail("skv_route_tokens", "groups must divide the experts, and the kept groups must hold the choices");
    const size_t smem = (size_t)(hidden + 2 * experts) * sizeof(float);
    auto kernel = route_tokens_kernel<skv_t>;
    if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return fail("skv_route_tokens", "the hidden size is too large");
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return fail("skv_route_tokens", "cannot reserve shared memory for a row");
    }
    return launch_pdl("skv_route_tokens", kernel, dim3(n), dim3(ROUTE_THREADS), smem, stream, (const skv_t*)h,
                      (const skv_t*)router, correction, (const skv_t*)shared_gate, hidden, experts, top, scale,
                      renormalize, chosen, weights, share, softmax, groups, keep, renorm_eps);
}

SKV_EXPORT int skv_sort_by_expert(const int* chosen, int pairs, int top, int experts, int* offsets, int* order,
                                  int* place, cudaStream_t stream) {
    if (experts <= 0 || experts > ROUTE_MAX_EXPERTS || top <= 0) return fail("skv_sort_by_expert", "1 to 1024 experts are served");
    if (pairs < 0 || !chosen || !offsets || !order || !place) return fail("skv_sort_by_expert", "the choice and places for the result are needed");
    return launch_pdl("skv_sort_by_expert", sort_by_expert_kernel, dim3(1), dim3(1024), 0, stream, chosen, pairs, top,
                      experts, offsets, order, place);
}

// a [a_rows, a_stride] and w [experts, N, K] in the compute dtype; rows int [pairs] or null (row p reads a[p]);
// out [pairs, N] float (out_is_float) or the compute dtype; act: an activation's code or -1 for none.
// gated: w is [experts, 2 N, K], tiles of 8 gate rows and their 8 up rows; out = act(gate . a) * (up . a).
// In bfloat16, rows that lie in sorted order already (rows null, a_stride = K) with K a multiple of 8 go to the
// tensor-memory GEMM's grouped form; `flag` is where its bounded waits report that they gave up.
SKV_EXPORT int skv_expert_linear(const void* a, int a_stride, int a_rows, const int* rows, const void* w,
                                 const int* offsets, void* out, int out_is_float, int pairs, int experts, int N, int K,
                                 int act, int gated, int* flag, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (experts <= 0 || experts > ROUTE_MAX_EXPERTS || N <= 0 || K <= 0 || a_stride < K || a_rows <= 0)
        return fail("skv_expert_linear", "sizes do not agree");
    if (!a || !w || !offsets || !out) return fail("skv_expert_linear", "rows, weights, offsets and a place for the result are needed");
    if (act >= ACT_SWIGLU_CLAMP) return fail("skv_expert_linear", "this activation is not served");
    if (gated && (act < 0 || N % 8 != 0)) return fail("skv_expert_linear", "a gated weight needs an activation and whole tiles of 8 rows");
#if SKV_DTYPE == SKV_BF16
    if (!rows && a_stride == K && K % 8 == 0 && a_rows >= pairs && !(((uintptr_t)a | (uintptr_t)w) & 15) &&
        (!gated || (!out_is_float && act != ACT_RELU2)))
        return grouped_linear_tcgen05(a, w, offsets, out, out_is_float, pairs, experts, gated ? 2 * N : N, K,
                                      gated ? (act_t)act : (act >= 0 ? ((act_t)act | ACT_ON_STORE) : (act_t)0), gated,
                                      flag, stream);
#endif
    const int row_tiles = (pairs + EXP_ROWS - 1) / EXP_ROWS + experts;       // no expert leaves more than one part tile
    if (row_tiles > 65535) return fail("skv_expert_linear", "too many rows for one launch");
    const dim3 grid((N + EXP_OUTS - 1) / EXP_OUTS, row_tiles);
    if (gated) {
        if (out_is_float)
            return launch_pdl("skv_expert_linear", expert_linear_kernel<skv_t, float, true>, grid, dim3(256), 0, stream,
                              (const skv_t*)a, a_stride, rows, (const skv_t*)w, offsets, (float*)out, experts, N, K, act);
        return launch_pdl("skv_expert_linear", expert_linear_kernel<skv_t, skv_t, true>, grid, dim3(256), 0, stream,
                          (const skv_t*)a, a_stride, rows, (const skv_t*)w, offsets, (skv_t*)out, experts, N, K, act);
    }
    if (out_is_float)
        return launch_pdl("skv_expert_linear", expert_linear_kernel<skv_t, float, false>, grid, dim3(256), 0, stream,
                          (const skv_t*)a, a_stride, rows, (const skv_t*)w, offsets, (float*)out, experts, N, K, act);
    return launch_pdl("skv_expert_linear", expert_linear_kernel<skv_t, skv_t, false>, grid, dim3(256), 0, stream,
                      (const skv_t*)a, a_stride, rows, (const skv_t*)w, offsets, (skv_t*)out, experts, N, K, act);
}

// out [pairs, K] = a[rows[p]] (compute dtype; K * element size a multiple of 16 bytes, both 16-byte aligned).
SKV_EXPORT int skv_gather_rows(const void* a, int a_stride, const int* rows, void* out, int pairs, int K,
                               cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (!a || !rows || !out || K <= 0 || a_stride < K) return fail("skv_gather_rows", "rows, their indices and a place for them are needed");
    if ((K * sizeof(skv_t)) % 16 || (a_stride * sizeof(skv_t)) % 16 || (((uintptr_t)a | (uintptr_t)out) & 15))
        return fail("skv_gather_rows", "rows must be whole 16-byte pieces");
    return launch_pdl("skv_gather_rows", gather_rows_kernel<skv_t>, dim3((pairs + 7) / 8), dim3(256), 0, stream,
                      (const skv_t*)a, a_stride, rows, (skv_t*)out, pairs, K);
}

SKV_EXPORT int skv_combine_experts(const float* results, const int* place, const float* weights, const float* shared,
                                   const float* share, float* x, int n, int hidden, int top, int add,
                                   cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hidden <= 0 || top <= 0 || top > ROUTE_MAX_TOP) return fail("skv_combine_experts", "1 to 16 choices a token are served");
    if (!results || !place || !weights || !x || (share && !shared))
        return fail("skv_combine_experts", "results, places, weights and the stream are needed");
    return launch_pdl("skv_combine_experts", combine_experts_kernel, dim3(n), dim3(256), 0, stream, results, place,
                      weights, shared, share, x, hidden, top, add);
}
