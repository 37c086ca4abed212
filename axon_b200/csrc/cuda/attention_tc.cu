// Causal grouped-query attention for prompt portions on the 5th-generation tensor cores
// (head size 128, bfloat16 in, float accumulation, softmax in float).
//
// A CTA owns up to 128 query rows of one (request, kv head): rows are (token, head of the
// group) pairs, token-major.  Queries, keys and values are gathered into shared memory in
// the 128-byte-swizzled layouts the MMA reads (keys and values row by row through the block
// table with cp.async, keys two tiles ahead, values one).  For every 64-key tile i:
//
//   S = Q K_i^T    tcgen05.mma, M 128, N 64, K 128, into tensor memory (64 columns);
//   softmax        a thread per row reads its 64 scores (tcgen05.ld), masks per element where
//                  the tile is not seen whole (causal, window), keeps a running maximum and
//                  sum, and writes P = exp2(s - m) as bfloat16 in operand layout to shared memory;
//   O += P V_i     tcgen05.mma, M 128, N 128, K 64, V read MN-major as it lies in the cache,
//                  accumulated in tensor memory (128 columns).
//
// The maximum m that the exponent uses lags the true one: O is rescaled (tensor memory load,
// multiply, store) only when a row's maximum has grown by more than 2^8, which after the
// first tiles is rare; the sum l uses the same m, so O / l is exact all the same.  One
// thread issues P V_i and then Q K_{i+1}^T behind it with one commit, so the tensor pipe
// runs the next scores while the threads are still busy with loads, and the chain per tile
// is MMA -> softmax -> MMA.  Waits on mbarriers are bounded (see tcgen05.cuh).
#include "tcgen05.cuh"

namespace axon {

constexpr int AT_BM = 128, AT_BN = 64, AT_HD = 128, AT_THREADS = 128;
constexpr float AT_LAZY = 8.f;      // log2 units a row's maximum may grow before O is rescaled

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

// How a thread addresses the 8 rows (tid/16 + 8j) of a 64-key tile that it copies.  When the
// page size divides 64 a row's place inside its page is the same in every tile, so it is
// computed once; other page sizes divide per row.
struct AtRowMap {
    int in_page[8];     // row's index inside its page (pages that divide 64)
    int page_of[8];     // row's page within the tile (pages that divide 64)
    int pages_per_tile; // 64 / page size, or 0 when the page size does not divide 64
    int last_page;      // logical page of the last key
};
template <bool CHECKED>
__device__ __forceinline__ void at_pages(int (&pg)[8], const AtRowMap& map, const PagedKv& kv, const int32_t* bt, int key0, int kv_len) {
    if (map.pages_per_tile) {
        const int first = (key0 / AT_BN) * map.pages_per_tile;
#pragma unroll
        for (int j = 0; j < 8; ++j) pg[j] = bt[min(first + map.page_of[j], map.last_page)];   // past the end: finite data, masked later
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) pg[j] = bt[min(key0 + (int)(threadIdx.x >> 4) + 8 * j, kv_len - 1) / kv.page_size];
    }
    // checked tables (a kernel variant of its own, see kv_layout.h): after all eight loads, so
    // that these stay in flight together
    if (CHECKED) {
#pragma unroll
        for (int j = 0; j < 8; ++j) pg[j] = kv.page(pg[j]);
    }
}
// One 64-key tile of K or V: two 8 KiB halves [dims 0..63 | 64..127][key][64 dims].  `src` points at
// this thread's 16-byte chunk of row 0 of the kv head in page 0; `dst` at its chunk of tile row tid/16.
__device__ __forceinline__ void at_load_tile(uint32_t dst, const __nv_bfloat16* src, const AtRowMap& map, const PagedKv& kv,
                                             const int (&pg)[8], int key0, int kv_len) {
    if (map.pages_per_tile) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            at_cp_async16(dst + j * 1024, src + (long long)pg[j] * kv.page_stride + map.in_page[j] * AT_HD);
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int pos = min(key0 + (int)(threadIdx.x >> 4) + 8 * j, kv_len - 1);
            at_cp_async16(dst + j * 1024, src + (long long)pg[j] * kv.page_stride + (pos % kv.page_size) * AT_HD);
        }
    }
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool CHECKED>
__global__ void __launch_bounds__(AT_THREADS, 2)
attention_tc_kernel(const AtParams p) {
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_dyn);
    constexpr uint32_t Q_BYTES = 2 * AT_BM * 128, KV_BYTES = 2 * AT_BN * 128, P_BYTES = AT_BM * 128;
    const uint32_t q_sm = base, k_sm = q_sm + Q_BYTES, v_sm = k_sm + 2 * KV_BYTES, p_sm = v_sm + 2 * KV_BYTES;
    const uint32_t bar_s = p_sm + P_BYTES;
    volatile uint32_t& tmem_slot = *reinterpret_cast<volatile uint32_t*>(smem_dyn + Q_BYTES + 4 * KV_BYTES + P_BYTES + 16);
    constexpr uint32_t TMEM_COLS = 256;          // S: columns 0..63, O: columns 64..191
    if (base & 1023u) {                          // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicMax(&g_tc_error, 100u);
        return;
    }

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
    const int t_begin = kv_lo / AT_BN, n_tiles = (kv_hi + AT_BN - 1) / AT_BN - t_begin;
    const int key_base = t_begin * AT_BN;

    if (threadIdx.x == 0) {
        mbar_init(bar_s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(bar_s + 16), "r"(TMEM_COLS) : "memory");
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
    // pg_v: pages of the tile whose V is copied next; pg_k: of the tile whose K is copied next
    int pg_v[8], pg_k[8];
    AtRowMap map;
    map.pages_per_tile = AT_BN % p.kv.page_size == 0 ? AT_BN / p.kv.page_size : 0;
    map.last_page = (kv_len - 1) / p.kv.page_size;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int r = (int)(threadIdx.x >> 4) + 8 * j;
        map.page_of[j] = r / p.kv.page_size;
        map.in_page[j] = r % p.kv.page_size;
    }
    const int32_t* bt = p.kv.block_table + (long long)slot * p.kv.table_stride;
    const int chunk = threadIdx.x & 15;
    // this thread's chunk of tile row tid/16 (rows 8 apart are 1024 bytes apart and swizzle alike)
    const uint32_t dst_off = (uint32_t)(chunk >> 3) * (AT_BN * 128) + sw128_offset((int)(threadIdx.x >> 4), chunk & 7);
    const __nv_bfloat16* k_src = p.pool + p.kv.entry_offset + (long long)kvh * p.kv.page_size * AT_HD + chunk * 8;
    const __nv_bfloat16* v_src = k_src + p.kv.v_offset;
    const uint32_t k_dst = k_sm + dst_off, v_dst = v_sm + dst_off;
    at_pages<CHECKED>(pg_v, map, p.kv, bt, key_base, kv_len);
    at_pages<CHECKED>(pg_k, map, p.kv, bt, key_base + AT_BN, kv_len);
    at_load_tile(k_dst, k_src, map, p.kv, pg_v, key_base, kv_len);
    at_load_tile(v_dst, v_src, map, p.kv, pg_v, key_base, kv_len);
    if (n_tiles > 1) at_load_tile(k_dst + KV_BYTES, k_src, map, p.kv, pg_k, key_base + AT_BN, kv_len);
    asm volatile("cp.async.commit_group;");
#pragma unroll
    for (int j = 0; j < 8; ++j) pg_v[j] = pg_k[j];
    at_pages<CHECKED>(pg_k, map, p.kv, bt, key_base + 2 * AT_BN, kv_len);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    fence_async_proxy();                         // what cp.async and st.shared wrote must be seen by the MMA
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_s = tmem_slot, tmem_o = tmem_slot + 64;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    constexpr uint32_t idesc_s = instr_desc(AT_BM, AT_BN);               // Q K^T: both K-major
    constexpr uint32_t idesc_o = instr_desc_b_mn(AT_BM, AT_HD);          // P V: V MN-major

    auto issue_scores = [&](uint32_t kt) {
#pragma unroll
        for (int k = 0; k < AT_HD / TC_UMMA_K; ++k) {
            const uint64_t da = smem_desc(q_sm + (uint32_t)(k >> 2) * (AT_BM * 128)) + (uint64_t)(2 * (k & 3));
            const uint64_t db = smem_desc(kt + (uint32_t)(k >> 2) * (AT_BN * 128)) + (uint64_t)(2 * (k & 3));
            umma(tmem_s, da, db, idesc_s, k ? 1u : 0u);
        }
    };
    if (threadIdx.x == 0) {
        issue_scores(k_sm);
        umma_commit(bar_s);
    }

    const int my_pos = row < rows_used ? pos0 + row / p.group : -1;      // unused rows see no key
    const int my_lo = p.window > 0 ? my_pos - p.window + 1 : 0;
    float m_use = -INFINITY, l = 0.f;            // the maximum the exponents use (log2 units), the running sum

    for (int it = 0; it < n_tiles; ++it) {
        const int buf = it & 1;
        const int key0 = key_base + it * AT_BN;
        mbar_wait(bar_s, it & 1, 0);             // S_it is there, and P V_{it-1} is done
        __syncwarp();
        tc_fence_after();
        // K_it and V_{it-1} are read: their buffers take K_{it+2} and V_{it+1}
        if (it + 2 < n_tiles) at_load_tile(k_dst + buf * KV_BYTES, k_src, map, p.kv, pg_k, key0 + 2 * AT_BN, kv_len);
        if (it + 1 < n_tiles) at_load_tile(v_dst + (buf ^ 1) * KV_BYTES, v_src, map, p.kv, pg_v, key0 + AT_BN, kv_len);
        asm volatile("cp.async.commit_group;");
#pragma unroll
        for (int j = 0; j < 8; ++j) pg_v[j] = pg_k[j];
        at_pages<CHECKED>(pg_k, map, p.kv, bt, key0 + 3 * AT_BN, kv_len);         // used in the next round

        // ---- this row's 64 scores
        uint32_t sr[2][32];
        tmem_ld32(tmem_s + lane_addr, sr[0]);
        tmem_ld32(tmem_s + lane_addr + 32, sr[1]);
        float mx0 = -INFINITY, mx1 = -INFINITY;
        const bool whole = key0 + AT_BN - 1 <= pos0 && (p.window <= 0 || key0 > pos0 + ntok - 1 - p.window);
        if (whole) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                mx0 = fmaxf(mx0, __uint_as_float(sr[0][i]));
                mx1 = fmaxf(mx1, __uint_as_float(sr[1][i]));
            }
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int kp = key0 + h * 32 + i;
                    const float v = (kp <= my_pos && kp >= my_lo) ? __uint_as_float(sr[h][i]) : -INFINITY;
                    sr[h][i] = __float_as_uint(v);
                    mx0 = fmaxf(mx0, v);
                }
        }
        const float m_new = fmaxf(m_use, fmaxf(mx0, mx1) * p.scale_log2);       // the scale is positive
        if (it == 0) {
            m_use = m_new;                       // nothing accumulated yet
        } else if (__any_sync(0xffffffffu, m_new > m_use + AT_LAZY)) {
            // the whole warp brings its rows of O to their new maxima (tensor memory access is per warp)
            const float corr = ex2(m_use - (m_new == -INFINITY ? 0.f : m_new));
            m_use = m_new;
            l *= corr;
#pragma unroll
            for (int c = 0; c < AT_HD / 32; ++c) {
                uint32_t orow[32];
                tmem_ld32(tmem_o + lane_addr + (uint32_t)(c * 32), orow);
#pragma unroll
                for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
                tmem_st32(tmem_o + lane_addr + (uint32_t)(c * 32), orow);
            }
            tmem_st_wait();
        }
        const float neg = m_use == -INFINITY ? 0.f : -m_use;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {              // 8 keys = one 16-byte chunk of the row of P
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = c * 8 + 2 * j;
                const float p0 = ex2(fmaf(__uint_as_float(sr[i >> 5][i & 31]), p.scale_log2, neg));
                const float p1 = ex2(fmaf(__uint_as_float(sr[(i + 1) >> 5][(i + 1) & 31]), p.scale_log2, neg));
                sum0 += p0;
                sum1 += p1;
                __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                pk[j] = *reinterpret_cast<uint32_t*>(&b);
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(p_sm + sw128_offset(row, c)), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]));
        }
        l += sum0 + sum1;
        asm volatile("cp.async.wait_group 1;" ::: "memory");     // V_it and K_{it+1} (the copies of the last round) landed
        fence_async_proxy();                     // P and the copies must be seen by the MMA
        tc_fence_before();
        __syncthreads();                         // all rows of P written, all scores read, O rescaled

        if (threadIdx.x == 0) {
            tc_fence_after();
            const uint32_t vt = v_sm + buf * KV_BYTES;
#pragma unroll
            for (int k = 0; k < AT_BN / TC_UMMA_K; ++k) {
                const uint64_t da = smem_desc(p_sm) + (uint64_t)(2 * k);
                // 16 keys = two groups of 8 along K: 2048 bytes further per step
                const uint64_t db = smem_desc_mn(vt + (uint32_t)k * 2048u, AT_BN * 128);
                umma(tmem_o, da, db, idesc_o, (it | k) ? 1u : 0u);
            }
            if (it + 1 < n_tiles) issue_scores(k_sm + (buf ^ 1) * KV_BYTES);
            umma_commit(bar_s);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    mbar_wait(bar_s, n_tiles & 1, 1);            // the last P V is done
    __syncwarp();
    tc_fence_after();

    {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int tok = q_start + tok0 + row / p.group, head = kvh * p.group + row % p.group;
        __nv_bfloat16* dst = p.out + ((long long)tok * p.heads + head) * AT_HD;
#pragma unroll
        for (int c = 0; c < AT_HD / 32; ++c) {
            uint32_t orow[32];
            tmem_ld32(tmem_o + lane_addr + (uint32_t)(c * 32), orow);     // by the whole warp, used rows or not
            if (row < rows_used) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint32_t pk[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(orow[v * 8 + 2 * j]) * inv,
                                                                 __uint_as_float(orow[v * 8 + 2 * j + 1]) * inv);
                        pk[j] = *reinterpret_cast<uint32_t*>(&b);
                    }
                    *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace axon

using namespace axon;

// Prompt portions at head size 128: tiles of `tokens_per_tile` tokens x group heads (<= 128 rows).
AXON_API int axon_attention_tc(const void* q, const void* pool, void* out, const int32_t* segments, int n_segments,
                               const int32_t* items, int n_items, const AxonKvLayout* layout, int heads, float scale,
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
    if (layout->planes == 1 || (layout->v_dim > 0 && layout->v_dim != AT_HD)) { set_error("axon_attention_tc: takes caches with key and value planes of one width"); return AXON_BAD_ARGUMENT; }
    p.kv = to_paged(layout);
    p.n_segments = n_segments; p.heads = heads; p.group = group; p.tokens_per_tile = tokens_per_tile; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    constexpr size_t smem = 2 * AT_BM * 128 + 4 * (2 * AT_BN * 128) + AT_BM * 128 + 64;
    if (p.kv.fault != nullptr) {
        if (int st = ensure_dynamic_smem<attention_tc_kernel<true>>(smem, "axon_attention_tc")) return st;
        attention_tc_kernel<true><<<dim3(n_items, kvh), AT_THREADS, smem, stream>>>(p);
    } else {
        if (int st = ensure_dynamic_smem<attention_tc_kernel<false>>(smem, "axon_attention_tc")) return st;
        attention_tc_kernel<false><<<dim3(n_items, kvh), AT_THREADS, smem, stream>>>(p);
    }
    return launch_status("axon_attention_tc");
}

AXON_API int axon_attention_tc_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof v) != cudaSuccess) return -1;
    return (int)v;
}
