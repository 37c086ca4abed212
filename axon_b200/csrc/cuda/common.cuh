// Shared device helpers for the engine's kernels (sm_100a).
//
// Element types: `float` for the true 32-bit path, `__nv_bfloat16` for serving.
// Reductions, softmax, norms, rotation and the residual stream are always float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pdl.cuh"

#define AXON_API extern "C" __attribute__((visibility("default")))

// Status codes returned by every launcher.
#define AXON_OK 0
#define AXON_BAD_ARGUMENT 1   // a size or pointer the kernel refuses (message via axon_last_error)
#define AXON_CUDA_ERROR 2     // the launch itself failed

namespace axon {

// The reason of the last refused call on this thread.
void set_error(const char* fmt, ...);

inline int launch_status(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return AXON_CUDA_ERROR;
    }
    return AXON_OK;
}

template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float ldf(const T* p) { return Elem<T>::load(p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v) { Elem<T>::store(p, v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions depends only on the block size, so a row's sum is the
// same whatever else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? smem32[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

// Where position `pos` of the request in `slot` lies: the element offset of row
// (kv_head, pos % page_size) of its page within one layer's K (or V) plane.
// Cache layout: pool[page][entry][2: K,V][kv_head][page_size][head_dim].
struct PagedKv {
    const int32_t* block_table;  // [slots][table_stride]: logical page -> physical page
    int table_stride;
    int page_size;
    int kv_heads;
    int head_dim;
    long long page_stride;   // elements between two pages of the pool
    long long entry_offset;  // elements from a page's start to this layer's K plane
    long long v_offset;      // elements from the K plane to the V plane

    __device__ __forceinline__ long long row(int slot, int pos, int kv_head) const {
        const int lp = pos / page_size;
        const int page = block_table[(long long)slot * table_stride + lp];
        return (long long)page * page_stride + entry_offset +
               ((long long)kv_head * page_size + (pos - lp * page_size)) * head_dim;
    }
};

}  // namespace axon
