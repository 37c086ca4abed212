// Causal grouped-query attention for prompt portions on the 5th-generation tensor cores
// (head size 128, bfloat16 in, float accumulation, softmax in float).
//
// A CTA (one per SM) owns up to 256 query rows of one (request, kv head): rows are (token, head
// of the group) pairs, token-major, in two sub-tiles of 128 rows that share every key and value
// tile.  Its warps have separate roles, so that the tensor pipe, the exponentials and the
// gathering of keys run at the same time instead of taking turns:
//
//   producers (2 warps)   gather 64-key tiles of K and of V row by row through the block table
//                         with cp.async into rings of shared memory, in the 128-byte-swizzled
//                         layout the MMA reads (K one tile ahead of V, two steps in flight);
//   MMA (2 threads)       one issues S = Q K_i^T (M 128, N 64, K 128) into one of a sub-tile's two
//                         score buffers in tensor memory, a tile ahead of the softmax; the other
//                         O += P V_i (M 128, N 128, K 64, V read MN-major as it lies in the cache)
//                         as soon as P is there; mbarriers (tcgen05.commit) tell the others;
//   softmax (2 x 4 warps) a thread per row reads its 64 scores (tcgen05.ld), masks per element
//                         where the tile is not seen whole (causal, window), keeps a running
//                         maximum and sum, and writes P = exp2(s - m) as bfloat16 back into
//                         tensor memory (tcgen05.st) over the first half of the scores it came
//                         from, where the value product reads it as its A operand: P never
//                         passes through shared memory, and the score buffer is free for the
//                         tile after the next once that value product is done.
//
// While one sub-tile's threads compute exponentials, the tensor pipe works on the other's
// products; neither waits for the gather.  The maximum m that the exponent uses lags the true
// one: O is rescaled (tensor memory load, multiply, store) only when a row's maximum has grown
// by more than 2^8, which after the first tiles is rare; the sum l uses the same m, so O / l is
// exact all the same.  Waits on mbarriers are bounded (see tcgen05.cuh): a wait that gives up
// sets the error flag and the kernel runs on to its end, where tensor memory is freed.
#include "tcgen05.cuh"

namespace axon {

constexpr int AT_BM = 128, AT_BN = 64, AT_HD = 128;
constexpr int AT_SUB = 2;                        // sub-tiles of 128 query rows per CTA
constexpr int AT_SOFTMAX_THREADS = AT_SUB * 128, AT_PRODUCERS = 64;
constexpr int AT_MMA_WARP = AT_SOFTMAX_THREADS / 32;                   // warp 8
constexpr int AT_PV_WARP = AT_MMA_WARP + 1 + AT_PRODUCERS / 32;        // warp 11
constexpr int AT_THREADS = AT_SOFTMAX_THREADS + 32 + AT_PRODUCERS + 32; // 8 softmax warps, the Q K^T warp, 2 producer warps, the P V warp
constexpr int AT_NK = 5, AT_NV = 5;              // stages of the key ring and of the value ring
constexpr float AT_LAZY = 8.f;                   // log2 units a row's maximum may grow before O is rescaled

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
template <int N> __device__ __forceinline__ void at_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The kernel's code is kept small on purpose: its three roles run different code at the same
// time, and an earlier version that unrolled every loop (155 KB of code) spent three cycles
// waiting for instructions for every one it issued.  Loops over the 64 scores of a row, over
// the 16 rows a producer thread copies and over the columns of O therefore stay loops.

// A producer thread copies one 16-byte chunk (`chunk` of the 16 of a row) of rows r0 + 4 j,
// j = 0..15, of one 64-key tile of K (plane 0) or V (plane = v_offset).  A tile is two 8 KiB
// halves [dims 0..63 | 64..127][key][64 dims], rows of 128 bytes with the 128-byte swizzle.
// Rows past the request's length read its last page or position: finite data, masked later.
struct AtGather {
    const int32_t* bt;          // the request's row of the block table
    const __nv_bfloat16* src;   // this thread's chunk of row 0 of the kv head in page 0 (key plane)
    long long page_stride;
    int ps, shift, kv_len, r0, last_page;
    bool quads;                 // the page size is a multiple of 16: rows 16 q .. 16 q + 15 of a tile share a page
    uint32_t dst0;              // byte offset of this thread's chunk within a tile's row 0, without the swizzle
    int chunk7;
};
// The pages of the four 16-row quarters of the tile that starts at key0 (page sizes that are
// multiples of 16).  Asked for a step ahead of the copies that need them: the copies of a step
// must not wait for the table, or the producers set the pace of the whole kernel.
template <bool CHECKED>
__device__ __forceinline__ void at_quad_pages(int (&pg)[4], const AtGather& g, const PagedKv& kv, int key0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) pg[q] = g.bt[min((key0 + 16 * q) / g.ps, g.last_page)];
    if (CHECKED) {
#pragma unroll
        for (int q = 0; q < 4; ++q) pg[q] = kv.page(pg[q]);
    }
}
__device__ __forceinline__ void at_copy_quads(const AtGather& g, const int (&pg)[4], uint32_t tile, int key0, long long plane) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int in_page = (key0 + 16 * q) % g.ps + g.r0;          // of the quarter's first row of this thread
        const __nv_bfloat16* from = g.src + plane + (long long)pg[q] * g.page_stride + in_page * AT_HD;
        const uint32_t to = tile + g.dst0 + (uint32_t)(16 * q + g.r0) * 128u;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)                             // rows 4 apart: 1 KiB further in the page, 512 bytes in the tile
            at_cp_async16(to + (uint32_t)jj * 512u + (uint32_t)((g.chunk7 ^ ((g.r0 + 4 * jj) & 7)) << 4), from + jj * 4 * AT_HD);
    }
}
// Any page size, row by row (each copy waits for its table entry).
template <bool CHECKED>
__device__ __forceinline__ void at_gather_rows(const AtGather& g, const PagedKv& kv, uint32_t tile, int key0, long long plane) {
#pragma unroll 4
    for (int j = 0; j < 16; ++j) {
        const int r = g.r0 + 4 * j;
        const int pos = min(key0 + r, g.kv_len - 1);
        const int lp = g.shift >= 0 ? pos >> g.shift : pos / g.ps;
        int page = g.bt[lp];
        if (CHECKED) page = kv.page(page);
        const __nv_bfloat16* from = g.src + plane + (long long)page * g.page_stride + (pos - lp * g.ps) * AT_HD;
        at_cp_async16(tile + g.dst0 + (uint32_t)r * 128u + (uint32_t)((g.chunk7 ^ (r & 7)) << 4), from);
    }
}

template <bool CHECKED>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tc_kernel(const AtParams p) {
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem_dyn);
    constexpr uint32_t QSUB_BYTES = 2 * AT_BM * 128;            // a sub-tile: two halves [dims 0..63 | 64..127][row][64 dims]
    constexpr uint32_t KV_BYTES = 2 * AT_BN * 128;              // a tile: two halves [dims 0..63 | 64..127][key][64 dims]
    const uint32_t q_sm = base, k_sm = q_sm + AT_SUB * QSUB_BYTES, v_sm = k_sm + AT_NK * KV_BYTES;
    const uint32_t bars = v_sm + AT_NV * KV_BYTES;
    // mbarriers, 8 bytes each; s_full, p_full and pv_done per (sub-tile, score buffer): a wait by
    // phase parity may lag its barrier by one phase only, and the softmax threads can be two tiles
    // ahead of the thread that issues P V
    const uint32_t k_full = bars, k_empty = k_full + 8 * AT_NK, v_full = k_empty + 8 * AT_NK, v_empty = v_full + 8 * AT_NV;
    const uint32_t s_full = v_empty + 8 * AT_NV, p_full = s_full + 16 * AT_SUB, pv_done = p_full + 16 * AT_SUB;
    const uint32_t tmem_slot_addr = pv_done + 16 * AT_SUB;      // (pv_done: per sub-tile and P buffer)
    volatile uint32_t& tmem_slot = *reinterpret_cast<volatile uint32_t*>(smem_dyn + (tmem_slot_addr - base));
    // tensor memory: two score buffers of 64 columns per sub-tile in columns 0..255, O of the sub-tiles in 256..383 and 384..511
    constexpr uint32_t TMEM_COLS = 512, TMEM_O = 2 * AT_SUB * AT_BN;
    if (base & 1023u) {                          // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicMax(&g_tc_error, 100u);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.y, kvh = blockIdx.x;              // the kv heads of an item side by side: items come longest first
    const int seg = p.items[2 * item], tok0 = p.items[2 * item + 1];
    const int slot = p.segments[seg], q_start = p.segments[p.n_segments + seg];
    const int q_len = p.segments[2 * p.n_segments + seg], kv_len = p.segments[3 * p.n_segments + seg];
    const int ntok = min(p.tokens_per_tile, q_len - tok0);
    const int rows_used = ntok * p.group;
    const int n_sub = rows_used > AT_BM ? 2 : 1;                // a short portion leaves the second sub-tile idle
    const int pos0 = kv_len - q_len + tok0;
    const int kv_hi = pos0 + ntok;
    const int kv_lo = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int t_begin = kv_lo / AT_BN, n_tiles = (kv_hi + AT_BN - 1) / AT_BN - t_begin;
    const int key_base = t_begin * AT_BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < AT_NK; ++s) { mbar_init(k_full + 8 * s, AT_PRODUCERS); mbar_init(k_empty + 8 * s, 1); }
        for (int s = 0; s < AT_NV; ++s) { mbar_init(v_full + 8 * s, AT_PRODUCERS); mbar_init(v_empty + 8 * s, 1); }
        for (int g = 0; g < AT_SUB; ++g) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(s_full + 16 * g + 8 * b, 1);
                mbar_init(p_full + 16 * g + 8 * b, 4);      // one arrival per softmax warp of the sub-tile
                mbar_init(pv_done + 16 * g + 8 * b, 1);
            }
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == AT_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tmem_slot_addr), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();                             // the barriers are initialised, tensor memory is there
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp > AT_MMA_WARP && warp < AT_PV_WARP) {
        // ================= producers.  Step j asks for K(j) and V(j - 1) (one commit group); two
        // a step stays in flight: when step j's copies are asked for, step j - 1's are waited for
        // and announced.
        const int tid = threadIdx.x - (AT_SOFTMAX_THREADS + 32);
        AtGather g;
        g.ps = p.kv.page_size; g.kv_len = kv_len;
        g.shift = (g.ps & (g.ps - 1)) == 0 ? 31 - __clz(g.ps) : -1;
        g.quads = g.ps % 16 == 0;
        g.last_page = (kv_len - 1) / g.ps;
        g.bt = p.kv.block_table + (long long)slot * p.kv.table_stride;
        const int chunk = tid & 15;
        g.r0 = tid >> 4;
        g.chunk7 = chunk & 7;
        g.src = p.pool + p.kv.entry_offset + (long long)kvh * p.kv.page_size * AT_HD + chunk * 8;
        g.page_stride = p.kv.page_stride;
        g.dst0 = (uint32_t)(chunk >> 3) * (AT_BN * 128);
        const long long v_plane = p.kv.v_offset;
        auto announce = [&](int j) {             // step j's copies have landed
            fence_async_proxy();
            if (j < n_tiles) mbar_arrive(k_full + 8 * (j % AT_NK));
            if (j >= 1) mbar_arrive(v_full + 8 * ((j - 1) % AT_NV));
        };
        // pages of tile j + 1 (asked for during step j), of tile j (its keys go now) and of tile j - 1 (its values go now)
        int pg_next[4] = {0, 0, 0, 0}, pg_k[4] = {0, 0, 0, 0}, pg_v[4] = {0, 0, 0, 0};
        if (g.quads) at_quad_pages<CHECKED>(pg_k, g, p.kv, key_base);
#pragma unroll 1
        for (int j = 0; j <= n_tiles; ++j) {
            if (g.quads && j + 1 < n_tiles) at_quad_pages<CHECKED>(pg_next, g, p.kv, key_base + (j + 1) * AT_BN);
            if (j < n_tiles) {
                if (j >= AT_NK) mbar_wait_idle(k_empty + 8 * (j % AT_NK), ((j / AT_NK) - 1) & 1, 3);
                const uint32_t tile = k_sm + (j % AT_NK) * KV_BYTES;
                if (g.quads) at_copy_quads(g, pg_k, tile, key_base + j * AT_BN, 0);
                else at_gather_rows<CHECKED>(g, p.kv, tile, key_base + j * AT_BN, 0);
            }
            if (j >= 1) {
                const int t = j - 1;
                if (t >= AT_NV) mbar_wait_idle(v_empty + 8 * (t % AT_NV), ((t / AT_NV) - 1) & 1, 3);
                const uint32_t tile = v_sm + (t % AT_NV) * KV_BYTES;
                if (g.quads) at_copy_quads(g, pg_v, tile, key_base + t * AT_BN, v_plane);
                else at_gather_rows<CHECKED>(g, p.kv, tile, key_base + t * AT_BN, v_plane);
            }
            asm volatile("cp.async.commit_group;");
            if (j >= 1) {
                at_cp_async_wait<1>();           // one step stays in flight
                announce(j - 1);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) { pg_v[q] = pg_k[q]; pg_k[q] = pg_next[q]; }
        }
        at_cp_async_wait<0>();
        announce(n_tiles);
    } else if (warp <= AT_MMA_WARP) {
        // ---- queries -> shared, by the softmax and MMA warps (the producers are already gathering keys); unused rows zero
#pragma unroll 1
        for (int e = threadIdx.x; e < AT_SUB * AT_BM * 16; e += AT_SOFTMAX_THREADS + 32) {
            const int R = e >> 4, c = e & 15;                       // R: row of the whole tile
            const int g = R >> 7, r = R & 127;
            const uint32_t dst = q_sm + (uint32_t)g * QSUB_BYTES + (uint32_t)(c >> 3) * (AT_BM * 128) + sw128_offset(r, c & 7);
            if (R < rows_used) {
                const int tok = q_start + tok0 + R / p.group, head = kvh * p.group + R % p.group;
                at_cp_async16(dst, p.q + ((long long)tok * p.heads + head) * AT_HD + c * 8);
            } else {
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u));
            }
        }
        asm volatile("cp.async.commit_group;");
        at_cp_async_wait<0>();
        fence_async_proxy();                     // what cp.async and st.shared wrote must be seen by the MMA
        tc_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFTMAX_THREADS + 32) : "memory");
        tc_fence_after();
    }

    if (warp == AT_MMA_WARP) {
        // ================= the thread that issues the score products (the value products have a
        // thread of their own, so that neither kind waits behind the other's barriers)
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc(AT_BM, AT_BN);               // Q K^T: both K-major
            // the scores of tile t of sub-tile g into its buffer t & 1
            auto issue_scores = [&](int g, int t, uint32_t kt) {
                const uint32_t qg = q_sm + (uint32_t)g * QSUB_BYTES;
                const uint32_t d = tmem + (uint32_t)((2 * g + (t & 1)) * AT_BN);
#pragma unroll
                for (int k = 0; k < AT_HD / TC_UMMA_K; ++k) {
                    const uint64_t da = smem_desc(qg + (uint32_t)(k >> 2) * (AT_BM * 128)) + (uint64_t)(2 * (k & 3));
                    const uint64_t db = smem_desc(kt + (uint32_t)(k >> 2) * (AT_BN * 128)) + (uint64_t)(2 * (k & 3));
                    umma(d, da, db, idesc_s, k ? 1u : 0u);
                }
                umma_commit(s_full + 16 * g + 8 * (t & 1));
            };
#pragma unroll 1
            for (int t = 0; t < n_tiles; ++t) {
                // tile t's scores go to buffer t & 1, which held the scores and then P of tile t - 2:
                // free once that tile's value product has read P
                const int ks = t % AT_NK;
                mbar_wait_idle(k_full + 8 * ks, (t / AT_NK) & 1, 1);
                for (int g = 0; g < n_sub; ++g) {
                    if (t >= 2) mbar_wait_idle(pv_done + 16 * g + 8 * (t & 1), ((t - 2) >> 1) & 1, 1);
                    tc_fence_after();
                    issue_scores(g, t, k_sm + ks * KV_BYTES);
                }
                umma_commit(k_empty + 8 * ks);
            }
        }
    } else if (warp == AT_PV_WARP) {
        // ================= the thread that issues O += P V
        if (lane == 0) {
            constexpr uint32_t idesc_o = instr_desc_b_mn(AT_BM, AT_HD);          // P V: V MN-major
#pragma unroll 1
            for (int i = 0; i < n_tiles; ++i) {
                const int vs = i % AT_NV;
                mbar_wait_idle(v_full + 8 * vs, (i / AT_NV) & 1, 4);
                const uint32_t vt = v_sm + vs * KV_BYTES;
                for (int g = 0; g < n_sub; ++g) {
                    mbar_wait_idle(p_full + 16 * g + 8 * (i & 1), (i >> 1) & 1, 4);
                    tc_fence_after();
                    // P lies in tensor memory, over the first half of the score buffer it came from
                    const uint32_t pt = tmem + (uint32_t)((2 * g + (i & 1)) * AT_BN);
#pragma unroll
                    for (int k = 0; k < AT_BN / TC_UMMA_K; ++k) {
                        // 16 keys = two groups of 8 along K: 2048 bytes further per step; 8 columns of P
                        const uint64_t db = smem_desc_mn(vt + (uint32_t)k * 2048u, AT_BN * 128);
                        umma_ta(tmem + TMEM_O + (uint32_t)(g * AT_HD), pt + (uint32_t)(8 * k), db, idesc_o, (i | k) ? 1u : 0u);
                    }
                    umma_commit(pv_done + 16 * g + 8 * (i & 1));
                }
                umma_commit(v_empty + 8 * vs);
            }
        }
    } else if (warp < 4 * n_sub) {
        // ================= softmax: warp w of sub-tile g owns tensor-memory lanes 32 (w % 4) ..
        const int g = warp >> 2;
        const int row = threadIdx.x & 127;                      // row of the sub-tile = tensor-memory lane
        const int R = g * AT_BM + row;                          // row of the whole tile
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tmem_o = tmem + TMEM_O + (uint32_t)(g * AT_HD) + lane_addr;
        const int my_pos = R < rows_used ? pos0 + R / p.group : -1;          // unused rows see no key
        const int my_lo = p.window > 0 ? my_pos - p.window + 1 : 0;
        // positions of the sub-tile's first and last used row: a tile all of them see whole needs no mask
        const int sub_first = pos0 + (g * AT_BM) / p.group;
        const int sub_last = pos0 + (min(rows_used, (g + 1) * AT_BM) - 1) / p.group;
        const bool all_rows_used = rows_used >= (g + 1) * AT_BM;
        float m_use = -INFINITY, l = 0.f;        // the maximum the exponents use (log2 units), the running sum

#pragma unroll 1
        for (int it = 0; it < n_tiles; ++it) {
            const int key0 = key_base + it * AT_BN;
            const uint32_t tmem_s = tmem + (uint32_t)((2 * g + (it & 1)) * AT_BN) + lane_addr;
            mbar_wait(s_full + 16 * g + 8 * (it & 1), (it >> 1) & 1, 0);
            __syncwarp();
            tc_fence_after();
            const bool whole = all_rows_used && key0 + AT_BN - 1 <= sub_first && (p.window <= 0 || key0 > sub_last - p.window);
            // ---- the row's 64 scores in two loads of 32 columns: the second is in flight while the first is used
            uint32_t sa[32], sb[32];
            tmem_ld32_issue(tmem_s, sa);
            tmem_ld32_issue(tmem_s + 32, sb);
            tmem_ld_wait();
            if (!whole) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int ka = key0 + i, kb = key0 + 32 + i;
                    if (!(ka <= my_pos && ka >= my_lo)) sa[i] = 0xff800000u;      // -inf
                    if (!(kb <= my_pos && kb >= my_lo)) sb[i] = 0xff800000u;
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                mx0 = fmaxf(mx0, __uint_as_float(sa[i]));
                mx1 = fmaxf(mx1, __uint_as_float(sa[i + 1]));
                mx2 = fmaxf(mx2, __uint_as_float(sb[i]));
                mx3 = fmaxf(mx3, __uint_as_float(sb[i + 1]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            const float m_new = fmaxf(m_use, mx * p.scale_log2);       // the scale is positive
            if (it == 0) {
                m_use = m_new;                   // nothing accumulated yet
            } else if (__any_sync(0xffffffffu, m_new > m_use + AT_LAZY)) {
                // the whole warp brings its rows of O to their new maxima (tensor memory access is per
                // warp); the product that last added to O must be through
                mbar_wait(pv_done + 16 * g + 8 * ((it - 1) & 1), ((it - 1) >> 1) & 1, 2);
                __syncwarp();
                tc_fence_after();
                const float corr = ex2(m_use - (m_new == -INFINITY ? 0.f : m_new));
                m_use = m_new;
                l *= corr;
#pragma unroll 1
                for (int c = 0; c < AT_HD / 32; ++c) {
                    uint32_t orow[32];
                    tmem_ld32(tmem_o + (uint32_t)(c * 32), orow);
#pragma unroll
                    for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
                    tmem_st32(tmem_o + (uint32_t)(c * 32), orow);
                }
                tmem_st_wait();
            }
            const float neg = m_use == -INFINITY ? 0.f : -m_use;
            // ---- P = exp2(s - m) as bfloat16 back into tensor memory, over the first 32 columns of
            // the scores it came from (a column holds two keys; the value product reads its A operand
            // there), and the row's sum
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
            for (int h = 0; h < 2; ++h) {            // keys 0..31, then 32..63: 16 columns of P each
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float s0 = __uint_as_float(h ? sb[2 * j] : sa[2 * j]), s1 = __uint_as_float(h ? sb[2 * j + 1] : sa[2 * j + 1]);
                    const float p0 = ex2(fmaf(s0, p.scale_log2, neg)), p1 = ex2(fmaf(s1, p.scale_log2, neg));
                    if (j & 1) { sum2 += p0; sum3 += p1; } else { sum0 += p0; sum1 += p1; }
                    __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                    pk[j] = *reinterpret_cast<uint32_t*>(&b);
                }
                tmem_st16(tmem_s + (uint32_t)(16 * h), pk);
            }
            sum0 += sum2; sum1 += sum3;
            l += sum0 + sum1;
            tmem_st_wait();                          // P (and a rescaled O) must be there before the MMA is told
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 16 * g + 8 * (it & 1));
        }
        mbar_wait(pv_done + 16 * g + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, 2);        // the last P V is done
        __syncwarp();
        tc_fence_after();
        {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const int tok = q_start + tok0 + R / p.group, head = kvh * p.group + R % p.group;
            __nv_bfloat16* dst = p.out + ((long long)tok * p.heads + head) * AT_HD;
#pragma unroll 1
            for (int c = 0; c < AT_HD / 32; ++c) {
                uint32_t orow[32];
                tmem_ld32(tmem_o + (uint32_t)(c * 32), orow);        // by the whole warp, used rows or not
                if (R < rows_used) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint32_t o4[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(orow[v * 8 + 2 * j]) * inv,
                                                                     __uint_as_float(orow[v * 8 + 2 * j + 1]) * inv);
                            o4[j] = *reinterpret_cast<uint32_t*>(&b);
                        }
                        *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == AT_MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace axon

using namespace axon;

// Prompt portions at head size 128: tiles of `tokens_per_tile` tokens x group heads (<= 256 rows).
AXON_API int axon_attention_tc(const void* q, const void* pool, void* out, const int32_t* segments, int n_segments,
                               const int32_t* items, int n_items, const AxonKvLayout* layout, int heads, float scale,
                               int window, int tokens_per_tile, cudaStream_t stream) {
    if (n_items <= 0) return AXON_OK;
    const int kvh = layout->kv_heads;
    if (layout->head_dim != AT_HD) { set_error("axon_attention_tc: head size %d is not 128", layout->head_dim); return AXON_BAD_ARGUMENT; }
    if (heads % kvh) { set_error("axon_attention_tc: %d heads over %d kv heads", heads, kvh); return AXON_BAD_ARGUMENT; }
    const int group = heads / kvh;
    if (tokens_per_tile < 1 || tokens_per_tile * group > AT_SUB * AT_BM) { set_error("axon_attention_tc: %d tokens x %d heads do not fit %d rows", tokens_per_tile, group, AT_SUB * AT_BM); return AXON_BAD_ARGUMENT; }
    if (((uintptr_t)q | (uintptr_t)pool | (uintptr_t)out) & 15) { set_error("axon_attention_tc: operands must be 16-byte aligned"); return AXON_BAD_ARGUMENT; }
    if (items == nullptr) { set_error("axon_attention_tc: needs a work list"); return AXON_BAD_ARGUMENT; }
    if (layout->planes == 1 || (layout->v_dim > 0 && layout->v_dim != AT_HD)) { set_error("axon_attention_tc: takes caches with key and value planes of one width"); return AXON_BAD_ARGUMENT; }
    AtParams p;
    p.q = (const __nv_bfloat16*)q; p.pool = (const __nv_bfloat16*)pool; p.out = (__nv_bfloat16*)out;
    p.segments = segments; p.items = items;
    p.kv = to_paged(layout);
    p.n_segments = n_segments; p.heads = heads; p.group = group; p.tokens_per_tile = tokens_per_tile; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    constexpr size_t smem = AT_SUB * 2 * AT_BM * 128 + (AT_NK + AT_NV) * (2 * AT_BN * 128) +
                            8 * (2 * AT_NK + 2 * AT_NV + 6 * AT_SUB) + 16;
    static_assert(smem <= 227 * 1024, "the tiles do not fit shared memory");
    if (p.kv.fault != nullptr) {
        if (int st = ensure_dynamic_smem<attention_tc_kernel<true>>(smem, "axon_attention_tc")) return st;
        attention_tc_kernel<true><<<dim3(kvh, n_items), AT_THREADS, smem, stream>>>(p);
    } else {
        if (int st = ensure_dynamic_smem<attention_tc_kernel<false>>(smem, "axon_attention_tc")) return st;
        attention_tc_kernel<false><<<dim3(kvh, n_items), AT_THREADS, smem, stream>>>(p);
    }
    return launch_status("axon_attention_tc");
}

// The largest tile this kernel takes, in query rows (tokens x heads of a group).
AXON_API int axon_attention_tc_rows() { return AT_SUB * AT_BM; }

AXON_API int axon_attention_tc_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof v) != cudaSuccess) return -1;
    return (int)v;
}
