// Picking tokens from logits on the device: argmax, repeat penalty, the k best
// candidates, and plain temperature sampling by inverse CDF.
//
// Order of candidates and ties follows the reference's sampler: a logit's key is
// its order-preserving bit pattern, NaN lowest, -0 equal to +0; among equal
// logits the larger id wins (src/sample.rs:280-305; argmax rule src/generate.rs:222-263).
#include "common.cuh"

namespace axon {

__device__ __forceinline__ uint32_t logit_key(float v) {
    if (v != v) return 0u;
    uint32_t b = (v == 0.0f) ? 0u : __float_as_uint(v);
    return (b >> 31) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_logit(uint32_t k) {
    return __uint_as_float((k >> 31) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ unsigned long long key64(float v, int id) {
    return ((unsigned long long)logit_key(v) << 32) | (unsigned)id;
}

__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* sm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long u = __shfl_xor_sync(0xffffffffu, v, o);
        v = u > v ? u : v;
    }
    __syncthreads();
    if (lane == 0) sm[warp] = v;
    __syncthreads();
    v = lane < nw ? sm[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long u = __shfl_xor_sync(0xffffffffu, v, o);
        v = u > v ? u : v;
    }
    return v;
}

// best[r] = the id of the largest logit of row r (last index among equal maxima;
// a NaN is picked only when the whole row is NaN, then the last index).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ best, int vocab,
                              long long row_stride) {
    __shared__ unsigned long long sm[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (long long)blockIdx.x * row_stride;
    unsigned long long k = 0;
    int tail = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // whole float4s, eight loads in flight per thread: the row's latency is paid once per
        // eight, not per element
        const int n4 = vocab >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        for (int i0 = threadIdx.x; i0 < n4; i0 += 8 * blockDim.x) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * blockDim.x;
                v[u] = i < n4 ? row4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * blockDim.x;
                if (i >= n4) continue;
                const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const unsigned long long c = key64(e[j], 4 * i + j);
                    k = c > k ? c : k;
                }
            }
        }
        tail = n4 << 2;
    }
    for (int i = tail + threadIdx.x; i < vocab; i += blockDim.x) {
        const unsigned long long c = key64(row[i], i);
        k = c > k ? c : k;
    }
    k = block_max_u64(k, sm);
    if (threadIdx.x == 0) best[blockIdx.x] = (int32_t)(k & 0xffffffffu);
}

// The repeat penalty on distinct ids: a positive logit is divided by p, any other
// multiplied (src/sample.rs:316-326).  ids: [rows][max_ids], -1 = none.
__global__ void penalty_kernel(float* __restrict__ logits, const int32_t* __restrict__ ids,
                               const float* __restrict__ penalty, int vocab, long long row_stride,
                               int max_ids) {
    const int r = blockIdx.x;
    const float p = penalty[r];
    if (p == 1.0f) return;
    for (int j = threadIdx.x; j < max_ids; j += blockDim.x) {
        const int id = ids[(long long)r * max_ids + j];
        if (id < 0 || id >= vocab) continue;
        float* v = logits + (long long)r * row_stride + id;
        *v = (*v > 0.0f) ? *v / p : *v * p;
    }
}

// The k (<= 256) best (logit, id) of each row, best first.  Radix select on the
// 64-bit key (logit key, id): keys are distinct, so exactly k pass the threshold.
constexpr int CAND_MAX = 256;

__global__ void __launch_bounds__(1024)
topk_kernel(const float* __restrict__ logits, const int32_t* __restrict__ ks,
            float* __restrict__ cand_logit, int32_t* __restrict__ cand_id, int vocab,
            long long row_stride) {
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long prefix_s;
    __shared__ int remaining_s;
    __shared__ unsigned long long picked[CAND_MAX];
    __shared__ int n_picked;
    const int r = blockIdx.x;
    const float* row = logits + (long long)r * row_stride;
    int k = ks[r];
    if (k > vocab) k = vocab;
    if (k > CAND_MAX) k = CAND_MAX;
    if (k <= 0) return;

    if (threadIdx.x == 0) { prefix_s = 0ull; remaining_s = k; n_picked = 0; }
    // digits of the key from the top: 4 bytes of logit key, then 4 bytes of id
    for (int shift = 56; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
        __syncthreads();
        const unsigned long long prefix = prefix_s;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const unsigned long long key = key64(row[i], i);
            if (shift == 56 || (key >> (shift + 8)) == prefix)
                atomicAdd(&hist[(key >> shift) & 0xff], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int rem = remaining_s;
            int d = 255;
            for (; d > 0; --d) {
                if ((int)hist[d] >= rem) break;
                rem -= (int)hist[d];
            }
            prefix_s = (prefix << 8) | (unsigned)d;
            remaining_s = rem;
        }
        __syncthreads();
    }
    const unsigned long long kth = prefix_s;  // the k-th largest key
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const unsigned long long key = key64(row[i], i);
        if (key >= kth) {
            const int at = atomicAdd(&n_picked, 1);
            if (at < CAND_MAX) picked[at] = key;
        }
    }
    __syncthreads();
    // pad and sort descending (bitonic over 256)
    for (int i = threadIdx.x; i < CAND_MAX; i += blockDim.x)
        if (i >= k) picked[i] = 0ull;
    __syncthreads();
    for (int size = 2; size <= CAND_MAX; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int i = threadIdx.x;
            if (i < CAND_MAX) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool desc = ((i & size) == 0);
                    const unsigned long long a = picked[i], b = picked[j];
                    if (desc ? (a < b) : (a > b)) { picked[i] = b; picked[j] = a; }
                }
            }
            __syncthreads();
        }
    }
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        cand_logit[(long long)r * CAND_MAX + i] = key_logit((uint32_t)(picked[i] >> 32));
        cand_id[(long long)r * CAND_MAX + i] = (int32_t)(picked[i] & 0xffffffffu);
    }
}

// Plain temperature sampling over the whole row: the token whose cumulative
// weight exp((l - max) / T) first passes u * total, ids ascending.  Sums are in
// double; each thread owns one contiguous stretch of the row.
__global__ void __launch_bounds__(1024)
sample_temperature_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                          const double* __restrict__ uniform, int32_t* __restrict__ picked, int vocab,
                          long long row_stride) {
    __shared__ float redf[32];
    __shared__ double part[1024];
    __shared__ double total_s;
    __shared__ int chosen;
    const int r = blockIdx.x;
    const float* row = logits + (long long)r * row_stride;
    const float inv_t = 1.0f / temperature[r];
    float m = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v == v) m = fmaxf(m, v);
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) redf[threadIdx.x >> 5] = m;
    __syncthreads();
    m = (threadIdx.x & 31) < ((blockDim.x + 31) >> 5) ? redf[threadIdx.x & 31] : -INFINITY;
    m = warp_max(m);

    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int lo = min(vocab, (int)threadIdx.x * per), hi = min(vocab, lo + per);
    double s = 0.0;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v == v) s += (double)expf((v - m) * inv_t);
    }
    part[threadIdx.x] = s;
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        double run = 0.0;
        for (int i = 0; i < (int)blockDim.x; ++i) { const double c = part[i]; part[i] = run; run += c; }
        total_s = run;
    }
    __syncthreads();
    const double total = total_s;
    double target = uniform[r] * total;
    if (target >= total) target = nextafter(total, 0.0);
    const double before = part[threadIdx.x];
    if (hi > lo && target >= before && target < before + s) {
        double cum = before;
        int pick = -1, last = -1;
        for (int i = lo; i < hi; ++i) {
            const float v = row[i];
            if (v != v) continue;
            const double w = (double)expf((v - m) * inv_t);
            if (w > 0.0) last = i;
            cum += w;
            if (target < cum) { pick = i; break; }
        }
        if (pick < 0) pick = last;
        if (pick >= 0) atomicMax(&chosen, pick);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int c = chosen;
        if (c < 0) {
            // rounding left the target between two stretches: take the last token with weight
            for (int i = vocab - 1; i >= 0; --i) {
                const float v = row[i];
                if (v == v && expf((v - m) * inv_t) > 0.f) { c = i; break; }
            }
            if (c < 0) c = vocab - 1;
        }
        picked[r] = c;
    }
}

}  // namespace axon

using namespace axon;

AXON_API int axon_argmax(const float* logits, int32_t* best, int rows, int vocab, long long row_stride,
                         cudaStream_t stream) {
    if (rows <= 0) return AXON_OK;
    if (vocab <= 0) { set_error("axon_argmax: empty rows"); return AXON_BAD_ARGUMENT; }
    launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, stream, logits, best, vocab, row_stride);
    return launch_status("axon_argmax");
}

AXON_API int axon_repeat_penalty(float* logits, const int32_t* ids, const float* penalty, int rows,
                                 int vocab, long long row_stride, int max_ids, cudaStream_t stream) {
    if (rows <= 0 || max_ids <= 0) return AXON_OK;
    penalty_kernel<<<rows, 64, 0, stream>>>(logits, ids, penalty, vocab, row_stride, max_ids);
    return launch_status("axon_repeat_penalty");
}

AXON_API int axon_topk_max() { return CAND_MAX; }

// cand_logit / cand_id: [rows][256]; ks[r] <= 256 entries of row r are written.
AXON_API int axon_topk(const float* logits, const int32_t* ks, float* cand_logit, int32_t* cand_id,
                       int rows, int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return AXON_OK;
    if (vocab <= 0) { set_error("axon_topk: empty rows"); return AXON_BAD_ARGUMENT; }
    topk_kernel<<<rows, 1024, 0, stream>>>(logits, ks, cand_logit, cand_id, vocab, row_stride);
    return launch_status("axon_topk");
}

AXON_API int axon_sample_temperature(const float* logits, const float* temperature,
                                     const double* uniform, int32_t* picked, int rows, int vocab,
                                     long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return AXON_OK;
    if (vocab <= 0) { set_error("axon_sample_temperature: empty rows"); return AXON_BAD_ARGUMENT; }
    sample_temperature_kernel<<<rows, 1024, 0, stream>>>(logits, temperature, uniform, picked, vocab, row_stride);
    return launch_status("axon_sample_temperature");
}
