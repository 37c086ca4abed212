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

// f(value, index) for every element of a row, each thread taking every blockDim-th float4 with
// eight loads in flight (rows that are not 16-byte aligned go element by element).
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int vocab, F f) {
    int tail = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
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
                if (i < n4) { f(v[u].x, 4 * i); f(v[u].y, 4 * i + 1); f(v[u].z, 4 * i + 2); f(v[u].w, 4 * i + 3); }
            }
        }
        tail = n4 << 2;
    }
    for (int i = tail + threadIdx.x; i < vocab; i += blockDim.x) f(row[i], i);
}

// hist[256] counts a digit; `rem` of the largest are still wanted.  Returns the digit in which
// the rem-th largest lies and takes the counts of the digits above it off `rem`.  One warp.
__device__ __forceinline__ int digit_of_rank(const unsigned int* hist, int& rem) {
    const int lane = threadIdx.x & 31;
    // lane l owns digits 255 - 8 l .. 248 - 8 l, from the top
    unsigned int mine[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { mine[j] = hist[255 - 8 * lane - j]; sum += mine[j]; }
    unsigned int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    const unsigned int before = incl - sum;                       // count in the digits above this lane's
    const unsigned int hit = __ballot_sync(0xffffffffu, incl >= (unsigned)rem);
    const int owner = hit ? __ffs(hit) - 1 : 31;
    int d = 0, r = rem;
    if (lane == owner) {
        r = rem - (int)before;
        int j = 0;
        for (; j < 7; ++j) {
            if ((int)mine[j] >= r) break;
            r -= (int)mine[j];
        }
        d = 255 - 8 * lane - j;
    }
    d = __shfl_sync(0xffffffffu, d, owner);
    rem = __shfl_sync(0xffffffffu, r, owner);
    return d;
}

// best[r] = the id of the largest logit of row r (last index among equal maxima;
// a NaN is picked only when the whole row is NaN, then the last index).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, const int32_t* __restrict__ row_index,
                              int32_t* __restrict__ best, int vocab, long long row_stride) {
    __shared__ unsigned long long sm[32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (long long)(row_index ? row_index[blockIdx.x] : blockIdx.x) * row_stride;
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

constexpr int TOPK_POOL = 4096;      // candidates of the deciding top byte that fit shared memory

// General form: eight passes over the whole row, one per byte of the key.  For rows whose
// deciding top byte holds more values than the pool (thousands of nearly equal logits).
__device__ void topk_select_general(const float* __restrict__ row, int vocab, int k, unsigned int* hist,
                                    unsigned long long* picked, int* n_picked, unsigned long long* prefix_s, int* remaining_s) {
    if (threadIdx.x == 0) { *prefix_s = 0ull; *remaining_s = k; *n_picked = 0; }
    for (int shift = 56; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
        __syncthreads();
        const unsigned long long prefix = *prefix_s;
        for_each_logit(row, vocab, [&](float v, int i) {
            const unsigned long long key = key64(v, i);
            if (shift == 56 || (key >> (shift + 8)) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
        });
        __syncthreads();
        if (threadIdx.x < 32) {
            int rem = *remaining_s;
            const int d = digit_of_rank(hist, rem);
            if (threadIdx.x == 0) { *prefix_s = (prefix << 8) | (unsigned)d; *remaining_s = rem; }
        }
        __syncthreads();
    }
    const unsigned long long kth = *prefix_s;  // the k-th largest key
    for_each_logit(row, vocab, [&](float v, int i) {
        const unsigned long long key = key64(v, i);
        if (key >= kth) {
            const int at = atomicAdd(n_picked, 1);
            if (at < CAND_MAX) picked[at] = key;
        }
    });
    __syncthreads();
}

// Two passes over the row: a histogram of the key's top byte (a counter array per warp, so that
// the many values of one byte do not queue on one counter) finds the byte in which the k-th
// largest lies; the second pass takes everything above that byte and pools the values of that
// byte in shared memory, where seven more passes over the few pooled keys settle the rest.
__global__ void __launch_bounds__(1024)
topk_kernel(const float* __restrict__ logits, const int32_t* __restrict__ row_index, const int32_t* __restrict__ ks,
            float* __restrict__ cand_logit, int32_t* __restrict__ cand_id, int vocab,
            long long row_stride) {
    extern __shared__ __align__(16) unsigned char topk_smem[];   // 32 KiB: per-warp histograms, then the pool
    unsigned int* warp_hist = reinterpret_cast<unsigned int*>(topk_smem);            // [32][256]
    unsigned long long* pool = reinterpret_cast<unsigned long long*>(topk_smem);       // [TOPK_POOL]
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long prefix_s;
    __shared__ int remaining_s, n_picked, n_pool;
    __shared__ unsigned long long picked[CAND_MAX];
    const int r = blockIdx.x, warp = threadIdx.x >> 5;
    const float* row = logits + (long long)(row_index ? row_index[r] : r) * row_stride;
    int k = ks[r];
    if (k > vocab) k = vocab;
    if (k > CAND_MAX) k = CAND_MAX;
    if (k <= 0) return;

    for (int i = threadIdx.x; i < 32 * 256; i += blockDim.x) warp_hist[i] = 0u;
    if (threadIdx.x == 0) { n_picked = 0; n_pool = 0; }
    __syncthreads();
    for_each_logit(row, vocab, [&](float v, int) { atomicAdd(&warp_hist[warp * 256 + (logit_key(v) >> 24)], 1u); });
    __syncthreads();
    for (int d = threadIdx.x; d < 256; d += blockDim.x) {
        unsigned int c = 0;
#pragma unroll 8
        for (int w = 0; w < 32; ++w) c += warp_hist[w * 256 + d];
        hist[d] = c;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        int rem = k;
        const int d = digit_of_rank(hist, rem);
        if (threadIdx.x == 0) { prefix_s = (unsigned long long)d; remaining_s = rem; }
    }
    __syncthreads();
    const unsigned int top = (unsigned int)prefix_s;
    const bool fits = hist[top] <= (unsigned)TOPK_POOL;
    if (fits) {
        for_each_logit(row, vocab, [&](float v, int i) {
            const unsigned int d = logit_key(v) >> 24;
            if (d > top) picked[atomicAdd(&n_picked, 1)] = key64(v, i);          // fewer than k of them
            else if (d == top) pool[atomicAdd(&n_pool, 1)] = key64(v, i);
        });
        __syncthreads();
        // the remaining seven bytes, over the pool only
        const int n = n_pool;
        for (int shift = 48; shift >= 0; shift -= 8) {
            for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
            __syncthreads();
            const unsigned long long prefix = prefix_s;
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const unsigned long long key = pool[i];
                if ((key >> (shift + 8)) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
            }
            __syncthreads();
            if (threadIdx.x < 32) {
                int rem = remaining_s;
                const int d = digit_of_rank(hist, rem);
                if (threadIdx.x == 0) { prefix_s = (prefix << 8) | (unsigned)d; remaining_s = rem; }
            }
            __syncthreads();
        }
        const unsigned long long kth = prefix_s;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const unsigned long long key = pool[i];
            if (key >= kth) {
                const int at = atomicAdd(&n_picked, 1);
                if (at < CAND_MAX) picked[at] = key;
            }
        }
        __syncthreads();
    } else {
        topk_select_general(row, vocab, k, hist, picked, &n_picked, &prefix_s, &remaining_s);
    }
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
sample_temperature_kernel(const float* __restrict__ logits, const int32_t* __restrict__ row_index,
                          const float* __restrict__ temperature,
                          const double* __restrict__ uniform, int32_t* __restrict__ picked, int vocab,
                          long long row_stride) {
    __shared__ float redf[32];
    __shared__ double part[1024];
    __shared__ double total_s;
    __shared__ int chosen;
    const int r = blockIdx.x;
    const float* row = logits + (long long)(row_index ? row_index[r] : r) * row_stride;
    const float inv_t = 1.0f / temperature[r];
    float m = -INFINITY;
    for_each_logit(row, vocab, [&](float v, int) { if (v == v) m = fmaxf(m, v); });
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) redf[threadIdx.x >> 5] = m;
    __syncthreads();
    m = (threadIdx.x & 31) < ((blockDim.x + 31) >> 5) ? redf[threadIdx.x & 31] : -INFINITY;
    m = warp_max(m);

    // stretches of whole float4s, so that a thread reads its stretch sixteen bytes at a time
    const int per = ((vocab + blockDim.x - 1) / blockDim.x + 3) & ~3;
    const int lo = min(vocab, (int)threadIdx.x * per), hi = min(vocab, lo + per);
    double s = 0.0;
    int i = lo;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
#pragma unroll 8
        for (; i + 4 <= hi; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            if (v.x == v.x) s += (double)expf((v.x - m) * inv_t);
            if (v.y == v.y) s += (double)expf((v.y - m) * inv_t);
            if (v.z == v.z) s += (double)expf((v.z - m) * inv_t);
            if (v.w == v.w) s += (double)expf((v.w - m) * inv_t);
        }
    }
    for (; i < hi; ++i) {
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

// dst[r] = src[row_index[r]] (whole rows of floats): the copy that the penalty may write into.
__global__ void gather_rows_kernel(const float* __restrict__ src, const int32_t* __restrict__ row_index,
                                   float* __restrict__ dst, int width, long long src_stride) {
    const float* from = src + (long long)(row_index ? row_index[blockIdx.y] : blockIdx.y) * src_stride;
    float* to = dst + (long long)blockIdx.y * width;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < width; i += gridDim.x * blockDim.x) to[i] = from[i];
}

}  // namespace axon

using namespace axon;

// dst [rows][width] contiguous; row_index (may be null: rows in order) picks the rows of src.
AXON_API int axon_gather_rows(const float* src, const int32_t* row_index, float* dst, int rows, int width,
                              long long src_stride, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return AXON_OK;
    const int bx = (width + 1023) / 1024 > 64 ? 64 : (width + 1023) / 1024;
    gather_rows_kernel<<<dim3(bx, rows), 256, 0, stream>>>(src, row_index, dst, width, src_stride);
    return launch_status("axon_gather_rows");
}

// In the three pickers below `row_index` (may be null) names the row of `logits` that output row r
// reads, so that a caller picks from some rows of a batch without copying them.
AXON_API int axon_argmax_rows(const float* logits, const int32_t* row_index, int32_t* best, int rows, int vocab,
                              long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return AXON_OK;
    if (vocab <= 0) { set_error("axon_argmax: empty rows"); return AXON_BAD_ARGUMENT; }
    launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, stream, logits, row_index, best, vocab, row_stride);
    return launch_status("axon_argmax");
}

AXON_API int axon_argmax(const float* logits, int32_t* best, int rows, int vocab, long long row_stride,
                         cudaStream_t stream) {
    if (rows <= 0) return AXON_OK;
    if (vocab <= 0) { set_error("axon_argmax: empty rows"); return AXON_BAD_ARGUMENT; }
    launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, stream, logits, (const int32_t*)nullptr, best, vocab, row_stride);
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
AXON_API int axon_topk(const float* logits, const int32_t* row_index, const int32_t* ks, float* cand_logit, int32_t* cand_id,
                       int rows, int vocab, long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return AXON_OK;
    if (vocab <= 0) { set_error("axon_topk: empty rows"); return AXON_BAD_ARGUMENT; }
    topk_kernel<<<rows, 1024, 32 * 1024, stream>>>(logits, row_index, ks, cand_logit, cand_id, vocab, row_stride);
    return launch_status("axon_topk");
}

AXON_API int axon_sample_temperature(const float* logits, const int32_t* row_index, const float* temperature,
                                     const double* uniform, int32_t* picked, int rows, int vocab,
                                     long long row_stride, cudaStream_t stream) {
    if (rows <= 0) return AXON_OK;
    if (vocab <= 0) { set_error("axon_sample_temperature: empty rows"); return AXON_BAD_ARGUMENT; }
    sample_temperature_kernel<<<rows, 1024, 0, stream>>>(logits, row_index, temperature, uniform, picked, vocab, row_stride);
    return launch_status("axon_sample_temperature");
}
