// Shared helpers of the sm_100a kernel library: dtype codes, error reporting,
// loads that widen to float, warp and block reductions.
//
// Every entry point is extern "C", takes raw device pointers and a stream, and
// returns 0 or a non-zero code after recording a message that
// skv_last_error() returns.  Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#define SKV_F32 0
#define SKV_BF16 1

// Each build of the library serves one compute dtype and one head size.
#ifndef SKV_DTYPE
#error "compile with -DSKV_DTYPE=0 (float) or 1 (bfloat16)"
#endif
#ifndef SKV_HEAD_DIM
#error "compile with -DSKV_HEAD_DIM=<head size, a multiple of 16>"
#endif
#if SKV_DTYPE == SKV_BF16
typedef __nv_bfloat16 skv_t;
#else
typedef float skv_t;
#endif

#define SKV_EXPORT extern "C" __attribute__((visibility("default")))

namespace skv {

inline char* error_buffer() {
    static thread_local char buffer[512] = {0};
    return buffer;
}

inline int fail(const char* what, const char* detail = "") {
    snprintf(error_buffer(), 512, "%s%s%s", what, detail[0] ? ": " : "", detail);
    return 1;
}

inline int check_launch(const char* kernel) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return fail(kernel, cudaGetErrorString(status));
    return 0;
}

// ---- programmatic dependent launch ------------------------------------------
// Kernels of a step are launched so that the next one may start while the
// previous one drains: it can fetch what does not depend on its predecessor
// (weights, tables) and then waits.  pdl_wait() returns once the preceding
// kernel on the stream has completed and its writes are visible; nothing that a
// predecessor writes may be read, and nothing a predecessor reads may be
// written, before it.  Set SKV_NO_PDL=1 in the environment to launch plainly.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

inline bool pdl_enabled() {
    static const bool enabled = [] {
        const char* off = getenv("SKV_NO_PDL");
        return !(off && off[0] == '1');
    }();
    return enabled;
}

template <typename... KernelArgs, typename... Args>
inline int launch_pdl(const char* name, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                      cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl_enabled() ? 1 : 0;
    const cudaError_t status = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
    if (status != cudaSuccess) return fail(name, cudaGetErrorString(status));
    return 0;
}

// Number of SMs of the current device (asked once per process; a process drives one kind of GPU).
inline int sm_count() {
    static const int count = [] {
        int device = 0, value = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || value <= 0)
            value = 1;
        return value;
    }();
    return count;
}

// Activations of a gated feed-forward's gate, chosen by the part's spec (ops.ACTIVATIONS has the names).
enum { ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_RELU2 = 2, ACT_SWIGLU_CLAMP = 3, ACT_COUNT = 4 };
// How an activation travels through the projection kernels: its code in the low 8 bits, ACT_ON_STORE above them, and
// in the high 32 bits the bits of one float that the activation may need (zero for those without a parameter, so a
// plain code compares equal to its enum).
typedef long long act_t;
__device__ __forceinline__ float act_param(act_t act) { return __int_as_float((int)(act >> 32)); }
// Added to an activation's code where a projection without a gate applies it to what it stores
// (out = act(a . w^T), the plain feed-forward): the store epilogues look for this bit.
constexpr int ACT_ON_STORE = 0x100;

// gelu(g) = g/2 * (1 + tanh(sqrt(2/pi) * (g + 0.044715 g^3))), the "tanh" form.
__device__ __forceinline__ float gelu_tanh(float g) {
    return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

// A gated unit with both branches clamped (ACT_SWIGLU_CLAMP, parameter `limit`): g' = min(g, limit),
// u' = clamp(u, -limit, limit), value g' * sigmoid(1.702 g') * (u' + 1).
constexpr float SWIGLU_CLAMP_ALPHA = 1.702f;
__device__ __forceinline__ float clamped_swiglu(float g, float u, float limit) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-SWIGLU_CLAMP_ALPHA * g)) * (u + 1.0f);
}

// relu(z)^2
__device__ __forceinline__ float relu_squared(float z) {
    const float r = fmaxf(z, 0.0f);
    return r * r;
}

// What a store epilogue writes for the accumulated value v: v itself, or (ACT_ON_STORE) its activation.
__device__ __forceinline__ float stored_value(float v, act_t act) {
    if (!(act & ACT_ON_STORE)) return v;
    const int code = (int)(act & 0xff);
    if (code == ACT_RELU2) return relu_squared(v);
    if (code == ACT_GELU_TANH) return gelu_tanh(v);
    return v / (1.0f + expf(-v));                     // silu
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Two optional terms of an attention kernel, both off when their pointer is null.
//   bias:  a table [num_heads][bias_len]; bias[h][d] is taken off the score of a key at distance d from the
//          query (a distance beyond the table reads its last entry).  The entries are in units of log2, that is the
//          natural bias times log2 e: the kernels that take a table keep their scores so (2^x by the special-function
//          unit).
//   gate:  the logit of (token t, head h) at gate[t * gate_stride + h]; the head's output is multiplied by its sigmoid.
//          With gate_per_element there is a logit for every number of the output, that of (token t, head h, number d)
//          at gate[t * gate_stride + h * head_dim + d].
//   softcap: c > 0 turns a score s into c * tanh(s / c) before the softmax (kernels that know it say so).
struct AttentionExtras {
    const float* bias;
    int bias_len;
    const float* gate;
    int gate_stride;
    float softcap;
    int gate_per_element;
    const float* sink;                 // [num_heads] or null: exp(sink[h]) counts once in the softmax's denominator
};

// tanh(x) = 1 - 2 / (1 + e^(2x)) with the special-function unit's exponential and reciprocal: an absolute error of a
// few 1e-7, which is what a capped score needs (tanh.approx's 2^-11 relative error would be 0.01 on a cap of 30).
__device__ __forceinline__ float tanh_by_exp2(float x) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 2.8853900817779268f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return fmaf(-2.0f, r, 1.0f);
}

__device__ __forceinline__ float gate_factor(const AttentionExtras& extras, size_t token, int head) {
    if (!extras.gate || extras.gate_per_element) return 1.0f;
    return 1.0f / (1.0f + expf(-extras.gate[token * extras.gate_stride + head]));
}

// The factor of one output number where the gate is per number (1 otherwise).
__device__ __forceinline__ float gate_element(const AttentionExtras& extras, size_t token, int head, int head_dim, int d) {
    if (!extras.gate || !extras.gate_per_element) return 1.0f;
    return 1.0f / (1.0f + expf(-extras.gate[token * extras.gate_stride + (size_t)head * head_dim + d]));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace skv
