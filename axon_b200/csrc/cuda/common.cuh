// Shared device helpers for the engine's kernels (sm_100a).
//
// Element types: `float` for the true 32-bit path, `__nv_bfloat16` for serving.
// Reductions, softmax, norms, rotation and the residual stream are always float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kv_layout.h"
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

// Partial products that a split-K product for few rows left in scratch for the kernel that
// reads its output: partial[((n / 128) * splits + s) * ntok + token][n % 128] holds slab s of
// output (token, n).  The reader adds the slabs in ascending order (so the sum does not
// depend on timing), then the bias; `partial == nullptr` means there is nothing to fold.
struct SplitFold {
    const float* partial;
    const float* bias;
    int splits, ntok;

    // All loads of a round of eight slabs are issued before the first is used: a reader pays one
    // trip to L2 for them, not one per slab (missing slabs add zeros, which changes nothing).
    __device__ __forceinline__ float at(int token, int n) const {
        const float* p = partial + ((long long)(n >> 7) * splits * ntok + token) * 128 + (n & 127);
        const long long step = (long long)ntok * 128;
        float v = 0.f;
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float t[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) t[q] = s0 + q < splits ? __ldcg(p + (s0 + q) * step) : 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) v += t[q];
        }
        if (bias) v += bias[n];
        return v;
    }
    // four consecutive outputs n .. n + 3 (n % 4 == 0, so they lie in one 128-row tile)
    __device__ __forceinline__ float4 at4(int token, int n) const {
        const float4* p = reinterpret_cast<const float4*>(partial + ((long long)(n >> 7) * splits * ntok + token) * 128 + (n & 127));
        const long long step = (long long)ntok * 32;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float4 t[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) t[q] = s0 + q < splits ? __ldcg(p + (s0 + q) * step) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int q = 0; q < 8; ++q) { v.x += t[q].x; v.y += t[q].y; v.z += t[q].z; v.w += t[q].w; }
        }
        if (bias) {
            const float4 b = *reinterpret_cast<const float4*>(bias + n);
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
        }
        return v;
    }
};

// Where position `pos` of the request in `slot` lies: the element offset of row
// (kv_head, pos % page_size) of its page within one layer's K (or V) plane.
// Cache layout: pool[page][entry][K plane | V plane], a plane being [kv_head][page_size][width]
// with width head_dim for keys and v_dim for values (see kv_layout.h).
struct PagedKv {
    const int32_t* block_table;  // [slots][table_stride]: logical page -> physical page
    int table_stride;
    int page_size;
    int kv_heads;
    int head_dim;
    long long page_stride;   // elements between two pages of the pool
    long long entry_offset;  // elements from a page's start to this layer's K plane
    long long v_offset;      // elements from the K plane to the V plane
    int v_dim;               // elements of a value row
    int planes;              // 2, or 1 when values are read from the key plane
    int n_pages;             // the sink page's index
    uint32_t* fault;         // checked tables: see kv_layout.h

    // A block-table entry as a kernel may follow it: itself, or with checked tables the sink
    // page when it lies outside the pool (recorded in `fault`).
    __device__ __forceinline__ int page(int entry) const {
        if (fault != nullptr && (unsigned)entry > (unsigned)n_pages) {
            fault[1] = (uint32_t)entry;
            fault[0] = 1u;
            return n_pages;
        }
        return entry;
    }
    __device__ __forceinline__ long long row(int slot, int pos, int kv_head) const {
        const int lp = pos / page_size;
        const int pg = page(block_table[(long long)slot * table_stride + lp]);
        return (long long)pg * page_stride + entry_offset +
               ((long long)kv_head * page_size + (pos - lp * page_size)) * head_dim;
    }
    // the same without the check, for kernels that have a variant of their own for checked tables
    // (a check may store, and a possible store keeps the compiler from issuing loads together)
    __device__ __forceinline__ long long row_unchecked(int slot, int pos, int kv_head) const {
        const int lp = pos / page_size;
        const int pg = block_table[(long long)slot * table_stride + lp];
        return (long long)pg * page_stride + entry_offset +
               ((long long)kv_head * page_size + (pos - lp * page_size)) * head_dim;
    }
    // the value row of the same position (from the pool's start, v_offset included)
    __device__ __forceinline__ long long v_row(int slot, int pos, int kv_head) const {
        const int lp = pos / page_size;
        const int pg = page(block_table[(long long)slot * table_stride + lp]);
        return (long long)pg * page_stride + entry_offset + v_offset +
               ((long long)kv_head * page_size + (pos - lp * page_size)) * v_dim;
    }
};

inline PagedKv to_paged(const AxonKvLayout* l) {
    PagedKv k;
    k.block_table = l->block_table;
    k.table_stride = l->table_stride;
    k.page_size = l->page_size;
    k.kv_heads = l->kv_heads;
    k.head_dim = l->head_dim;
    k.page_stride = l->page_stride;
    k.entry_offset = l->entry_offset;
    k.v_offset = l->v_offset;
    k.v_dim = l->v_dim > 0 ? l->v_dim : l->head_dim;
    k.planes = l->planes == 1 ? 1 : 2;
    k.n_pages = l->n_pages;
    k.fault = l->fault;
    return k;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize for a kernel, once per device (the attribute
// belongs to the device's context, so a second GPU needs its own call).
template <auto Kernel>
inline int ensure_dynamic_smem(size_t bytes, const char* what) {
    static bool done[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_error("%s: no current device", what); return AXON_CUDA_ERROR; }
    if (!done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) { set_error("%s: %s", what, cudaGetErrorString(e)); return AXON_CUDA_ERROR; }
        done[dev] = true;
    }
    return AXON_OK;
}

}  // namespace axon
