// Shared pieces of the sequence-model kernels (hybrid stacks of attention / recurrent mixers with routed feed-forwards): element types,
// the flat ragged batch every kernel indexes, small reductions.  Storage type T is __nv_bfloat16 or float (the all-32-bit mode); residual
// stream, norms, softmax, rotary angles, routers and recurrent state are float in both.
#pragma once
#include "../common.cuh"

namespace wf {
namespace seq {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// One step's ragged batch: n tokens laid out sequence after sequence.  All arrays live on the device.
struct Batch {
    int n = 0;                 // tokens
    int nseq = 0;              // sequences
    const int32_t* tok_seq;    // [n] index of the token's sequence in this step
    const int32_t* tok_pos;    // [n] absolute position in its sequence
    const int32_t* seq_start;  // [nseq] first token of the sequence in the flat batch
    const int32_t* seq_len;    // [nseq] tokens of the sequence in this step
    const int32_t* seq_pos0;   // [nseq] position of its first token
    const int32_t* seq_slot;   // [nseq] state slot = block-table row
    int max_len = 0;           // longest portion of the step (known on the host; sizes grids that cut portions into chunks)
};

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
// sum over a block of up to 1024 threads; every thread gets the result.  scratch: 33 floats of shared memory
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) scratch[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

}  // namespace seq
}  // namespace wf
