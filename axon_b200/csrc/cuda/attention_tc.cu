// Causal grouped-query attention for prompt portions on the 5th-generation tensor cores
// (head size 128, bfloat16 in, float accumulation, softmax in float).
//
// A CTA owns up to 128 query rows of one (request, kv head): rows are (token, head of the
// group) pairs, token-major.  Queries, keys and values are gathered into shared memory in
// the 128-byte-swizzled layouts the MMA reads (keys and values row by row through the block
// table with cp.async, two tiles deep).  For every 64-key tile:
//
//   S = Q K^T      tcgen05.mma, M 128, N 64, K 128, into tensor memory (64 columns);
//   softmax        a thread per row reads its 64 scores (tcgen05.ld), masks per element
//                  (causal, window), keeps a running maximum and sum, and writes
//                  P = exp2(s - m) as bfloat16 in operand layout over the tile's keys;
//   T = P V        tcgen05.mma, M 128, N 128, K 64, V read MN-major as it lies in the cache,
//                  into tensor memory (128 columns), then O = O * corr + T in registers.
//
// The accumulator of a row lives in its thread's registers, so rescaling needs no tensor
// memory round trip.  Waits on mbarriers are bounded (see tcgen05.cuh).
#include "tcgen05.cuh"

namespace axon {

constexpr int AT_BM = 128, AT_BN = 64, AT_HD = 128, AT_THREADS = 128;

struct AtParams {
    const __nv_bfloat16* q;      // [tokens][heads * 128]
    const __nv_bfloat16* pool;
    __nv_bfloat16* out;
    const int32_t* segments;     // [4][n_segments]: slot, q_start, q_len, kv_len
    const int32_t* items;        // [n_items][2]: segment, first token of the tile within the segment
    PagedKv kv;
    int n_segments, heads, group, tokens_per_tile, window;
    float scale_log2;
};

__device__ __forceinline__ void at_cp_async16(uint32_t smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(gmem));
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One 64-key tile of K and V: each as two 8 KiB halves [dims 0..63 | 64..127][key][64 dims].
__device__ __forceinline__ void at_load_kv(uint32_t k_tile, uint32_t v_tile, const __nv_bfloat16* pool, const PagedKv& kv,
                                           int slot, int kvh, int key0, int kv_len) {
    for (int e = threadIdx.x; e < AT_BN * 16; e += AT_THREADS) {
        const int r = e >> 4, c = e & 15;
        int pos = key0 + r;
        if (pos >= kv_len) pos = kv_len - 1;       // finite data, masked later
        const __nv_bfloat16* src = pool + kv.row(slot, pos, kvh) + c * 8;
        const uint32_t off = (uint32_t)(c >> 3) * (AT_BN * 128) + sw128_offset(r, c & 7);
        at_cp_async16(k_tile + off, src);
        at_cp_async16(v_tile + off, src + kv.v_offset);
    }
}

__global__ void __launch_bounds__(AT_THREADS, 2)
attention_tc_kernel(const AtParams p) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = ((uint32_t)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    constexpr uint32_t Q_BYTES = 2 * AT_BM * 128, KV_BYTES = 2 * AT_BN * 128;
    const uint32_t q_sm = base, k_sm = q_sm + Q_BYTES, v_sm = k_sm + 2 * KV_BYTES;
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_slot;
    const uint32_t bar_s = (uint32_t)__cvta_generic_to_shared(&bars[0]), bar_o = bar_s + 8;
    constexpr uint32_t TMEM_COLS = 256;          // S: columns 0..63, T: columns 64..191

    const int warp = threadIdx.x >> 5;
    const int row = threadIdx.x;                 // this thread's query row = its tensor-memory lane
    const int item = blockIdx.x, kvh = blockIdx.y;
    const int seg = p.items[2 * item], tok0 = p.items[2 * item + 1];
    const int slot = p.segments[seg], q_start = p.segments[p.n_segments + seg];
    const int q_len = p.segments[2 * p.n_segments + seg], kv_len = p.segments[3 * p.n_segments + seg];
    const int ntok = min(p.tokens_per_tile, q_len - tok0);
    const int rows_used = ntok * p.group;
    const int pos0 = kv_len - q_len + tok0;
    const int kv_hi = pos0 + ntok;
    const int kv_lo = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int t_begin = kv_lo / AT_BN, t_end = (kv_hi + AT_BN - 1) / AT_BN;

    if (threadIdx.x == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // ---- queries -> shared: two halves [dims 0..63 | 64..127][row][64 dims]; unused rows zero
    for (int e = threadIdx.x; e < AT_BM * 16; e += AT_THREADS) {
        const int r = e >> 4, c = e & 15;
        const uint32_t dst = q_sm + (uint32_t)(c >> 3) * (AT_BM * 128) + sw128_offset(r, c & 7);
        if (r < rows_used) {
            const int tok = q_start + tok0 + r / p.group, head = kvh * p.group + r % p.group;
            at_cp_async16(dst, p.q + ((long long)tok * p.heads + head) * AT_HD + c * 8);
        } else {
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u));
        }
    }
    at_load_kv(k_sm, v_sm, p.pool, p.kv, slot, kvh, t_begin * AT_BN, kv_len);
    asm volatile("cp.async.commit_group;");

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = tmem_slot, tmem_t = tmem_slot + 64;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;

    const int my_pos = row < rows_used ? pos0 + row / p.group : -1;      // unused rows see no key
    const int my_lo = p.window > 0 ? my_pos - p.window + 1 : 0;
    float o[AT_HD];
#pragma unroll
    for (int i = 0; i < AT_HD; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    constexpr uint32_t idesc_s = instr_desc(AT_BM, AT_BN);               // Q K^T: both K-major
    constexpr uint32_t idesc_t = instr_desc_b_mn(AT_BM, AT_HD);          // P V: V MN-major

    for (int tile = t_begin; tile < t_end; ++tile) {
        const int it = tile - t_begin, buf = it & 1;
        const uint32_t kt = k_sm + buf * KV_BYTES, vt = v_sm + buf * KV_BYTES;
        // P (128 rows x 64 keys, 16 KiB) takes the place of this tile's keys once S is computed:
        // the next load into this buffer is issued only after the P V product has been waited for
        const uint32_t p_sm = kt;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        fence_async_proxy();                     // what cp.async wrote must be seen by the MMA
        __syncthreads();                         // tile landed for all; everyone is done with the other buffer
        if (threadIdx.x == 0) {
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < AT_HD / TC_UMMA_K; ++k) {
                const uint64_t da = smem_desc(q_sm + (uint32_t)(k >> 2) * (AT_BM * 128)) + (uint64_t)(2 * (k & 3));
                const uint64_t db = smem_desc(kt + (uint32_t)(k >> 2) * (AT_BN * 128)) + (uint64_t)(2 * (k & 3));
                umma(tmem_s, da, db, idesc_s, k ? 1u : 0u);
            }
            umma_commit(bar_s);
        }
        // the next tile's loads run under this tile's products and softmax
        if (tile + 1 < t_end)
            at_load_kv(k_sm + (buf ^ 1) * KV_BYTES, v_sm + (buf ^ 1) * KV_BYTES, p.pool, p.kv, slot, kvh, (tile + 1) * AT_BN, kv_len);
        asm volatile("cp.async.commit_group;");
        mbar_wait(bar_s, it & 1, 0);
        __syncwarp();
        tc_fence_after();

        // ---- this row's 64 scores: running maximum and sum, P to shared memory.  Tiles that
        // every row of the CTA sees whole (most of them) skip the per-element mask.
        uint32_t sr[2][32];
        tmem_ld32(tmem_s + lane_addr, sr[0]);
        tmem_ld32(tmem_s + lane_addr + 32, sr[1]);
        float mx = -INFINITY;
        const int key0 = tile * AT_BN;
        const bool whole = key0 + AT_BN - 1 <= pos0 && (p.window <= 0 || key0 > pos0 + ntok - 1 - p.window);
        if (whole) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sr[h][i]));
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int kp = key0 + h * 32 + i;
                    const float v = (kp <= my_pos && kp >= my_lo) ? __uint_as_float(sr[h][i]) : -INFINITY;
                    sr[h][i] = __float_as_uint(v);
                    mx = fmaxf(mx, v);
                }
        }
        // m and l are kept in units of log2: score * scale_log2 (the scale is positive)
        const float m_new = fmaxf(m, mx * p.scale_log2);
        const float use = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = exp2f(m - use);
        const bool rescale = m_new != m;
        m = m_new;
        float sum = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {              // 8 keys = one 16-byte chunk of the row of P
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = c * 8 + 2 * j;
                const float p0 = exp2f(fmaf(__uint_as_float(sr[i >> 5][i & 31]), p.scale_log2, -use));
                const float p1 = exp2f(fmaf(__uint_as_float(sr[(i + 1) >> 5][(i + 1) & 31]), p.scale_log2, -use));
                sum += p0 + p1;
                __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                pk[j] = *reinterpret_cast<uint32_t*>(&b);
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(p_sm + sw128_offset(row, c)), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]));
        }
        fence_async_proxy();                     // P must be seen by the MMA
        tc_fence_before();
        __syncthreads();                         // all rows of P written, all scores read

        if (threadIdx.x == 0) {
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < AT_BN / TC_UMMA_K; ++k) {
                const uint64_t da = smem_desc(p_sm) + (uint64_t)(2 * k);
                // 16 keys = two groups of 8 along K: 2048 bytes further per step
                const uint64_t db = smem_desc_mn(vt + (uint32_t)k * 2048u, AT_BN * 128);
                umma(tmem_t, da, db, idesc_t, k ? 1u : 0u);
            }
            umma_commit(bar_o);
        }
        // the old accumulator is rescaled while the product runs (skipped by warps whose maxima stood)
        l = l * corr + sum;
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int i = 0; i < AT_HD; ++i) o[i] *= corr;
        }
        mbar_wait(bar_o, it & 1, 1);
        __syncwarp();
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < AT_HD / 32; ++c) {
            uint32_t tr[32];
            tmem_ld32(tmem_t + lane_addr + (uint32_t)(c * 32), tr);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(tr[i]);
        }
        tc_fence_before();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    if (row < rows_used) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int tok = q_start + tok0 + row / p.group, head = kvh * p.group + row % p.group;
        __nv_bfloat16* dst = p.out + ((long long)tok * p.heads + head) * AT_HD;
#pragma unroll
        for (int c = 0; c < AT_HD / 8; ++c) {
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 b = __floats2bfloat162_rn(o[c * 8 + 2 * j] * inv, o[c * 8 + 2 * j + 1] * inv);
                pk[j] = *reinterpret_cast<uint32_t*>(&b);
            }
            *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace axon

using namespace axon;

struct AxonKvLayoutTc {
    const int32_t* block_table;
    int32_t table_stride, page_size, kv_heads, head_dim;
    int64_t page_stride, entry_offset, v_offset;
};

// Prompt portions at head size 128: tiles of `tokens_per_tile` tokens x group heads (<= 128 rows).
AXON_API int axon_attention_tc(const void* q, const void* pool, void* out, const int32_t* segments, int n_segments,
                               const int32_t* items, int n_items, const AxonKvLayoutTc* layout, int heads, float scale,
                               int window, int tokens_per_tile, cudaStream_t stream) {
    if (n_items <= 0) return AXON_OK;
    const int kvh = layout->kv_heads;
    if (layout->head_dim != AT_HD) { set_error("axon_attention_tc: head size %d is not 128", layout->head_dim); return AXON_BAD_ARGUMENT; }
    if (heads % kvh) { set_error("axon_attention_tc: %d heads over %d kv heads", heads, kvh); return AXON_BAD_ARGUMENT; }
    const int group = heads / kvh;
    if (tokens_per_tile < 1 || tokens_per_tile * group > AT_BM) { set_error("axon_attention_tc: %d tokens x %d heads do not fit 128 rows", tokens_per_tile, group); return AXON_BAD_ARGUMENT; }
    if (((uintptr_t)q | (uintptr_t)pool | (uintptr_t)out) & 15) { set_error("axon_attention_tc: operands must be 16-byte aligned"); return AXON_BAD_ARGUMENT; }
    if (items == nullptr) { set_error("axon_attention_tc: needs a work list"); return AXON_BAD_ARGUMENT; }
    AtParams p;
    p.q = (const __nv_bfloat16*)q; p.pool = (const __nv_bfloat16*)pool; p.out = (__nv_bfloat16*)out;
    p.segments = segments; p.items = items;
    p.kv.block_table = layout->block_table; p.kv.table_stride = layout->table_stride; p.kv.page_size = layout->page_size;
    p.kv.kv_heads = kvh; p.kv.head_dim = AT_HD; p.kv.page_stride = layout->page_stride;
    p.kv.entry_offset = layout->entry_offset; p.kv.v_offset = layout->v_offset;
    p.n_segments = n_segments; p.heads = heads; p.group = group; p.tokens_per_tile = tokens_per_tile; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    constexpr size_t smem = 2 * AT_BM * 128 + 4 * (2 * AT_BN * 128) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error("axon_attention_tc: %s", cudaGetErrorString(e)); return AXON_CUDA_ERROR; }
        configured = true;
    }
    attention_tc_kernel<<<dim3(n_items, kvh), AT_THREADS, smem, stream>>>(p);
    return launch_status("axon_attention_tc");
}

AXON_API int axon_attention_tc_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof v) != cudaSuccess) return -1;
    return (int)v;
}
