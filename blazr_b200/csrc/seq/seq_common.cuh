// seq_common.cuh -- shared helpers of libb200seq (dense linear layers + sequence operators, sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/b200seq.h"

namespace b200seq {

void count_launch(int n = 1);
int fail(int code, const char* fmt, ...);
int cuda_status(cudaError_t e, const char* what);
int* error_flag_dev();   // device int: bit 0 = KV position outside the block table, bit 1 = bounded wait ran out, bit 2 = expert table entry out of range

#define SEQ_LAUNCH_CHECK(what)                         \
    do {                                               \
        cudaError_t e_ = cudaGetLastError();           \
        if (e_ != cudaSuccess) return cuda_status(e_, what); \
        count_launch();                                \
    } while (0)

__device__ __forceinline__ void store_act(void* out, int dtype, int64_t idx, float v) {
    if (dtype == B200SEQ_F32) reinterpret_cast<float*>(out)[idx] = v;
    else reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// sum over the block; every thread gets the result.  red: >= 33 floats of shared memory.  Fixed order: deterministic.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();   // red may still be read from the previous call
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ float sigmoidf_acc(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float siluf_acc(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_acc(float x) { return x > 20.f ? x : log1pf(expf(x)); }


// activation of a projection (include/b200seq.h: B200SEQ_ACT_*)
struct ActParams {
    int kind;
    float limit, alpha, shift;
};
__device__ __forceinline__ bool act_is_gated(int kind) { return kind == B200SEQ_ACT_SWISH_CLAMP || kind == B200SEQ_ACT_GELU_TANH; }
__device__ __forceinline__ float gelu_tanhf_acc(float z) { return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }
__device__ __forceinline__ float act_gated(const ActParams& a, float gate, float up) {
    if (a.kind == B200SEQ_ACT_GELU_TANH) return gelu_tanhf_acc(gate) * up;
    const float g = fminf(gate, a.limit);
    const float u = fminf(fmaxf(up, -a.limit), a.limit);
    return g * sigmoidf_acc(a.alpha * g) * (u + a.shift);
}
__device__ __forceinline__ float act_plain(int kind, float z) {
    if (kind == B200SEQ_ACT_RELU2) {
        const float r = fmaxf(z, 0.f);
        return r * r;
    }
    return z;
}
inline bool act_kind_gated(int kind) { return kind == B200SEQ_ACT_SWISH_CLAMP || kind == B200SEQ_ACT_GELU_TANH; }
inline bool act_kind_known(int kind) { return kind >= B200SEQ_ACT_SWISH_CLAMP && kind <= B200SEQ_ACT_IDENT; }

}  // namespace b200seq
