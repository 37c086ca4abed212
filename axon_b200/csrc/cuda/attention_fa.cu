// Causal grouped-query attention over the paged cache on the tensor cores
// (bfloat16 in, float accumulation, softmax in float).
//
// One kernel, two shapes of work:
//
//  * prefill: a CTA owns up to 64 query rows of one (request, kv head): rows are
//    (token, head of the group) pairs, token-major, so all heads of a group share the
//    keys they read.  Its 4 warps own 16 rows each and sweep 64-key tiles.
//  * decode: a CTA owns up to 16 query rows (one token's group of heads, or a few
//    tokens') and a contiguous share ("split") of the key tiles; inside a tile each
//    warp takes 16 of the 64 keys and the warps merge at the end.  With more than one
//    split the CTA writes an unnormalised partial (o, m, l) to scratch; the splits are
//    folded in ascending order either by the CTA that finishes last (when the caller
//    gives arrival counters) or by a second kernel.
//
// Keys and values are gathered row by row through the block table (any page size)
// with 16-byte cp.async into swizzled shared tiles, two (prefill) or three (decode) deep.  A row of a
// tile is one key of one kv head (head_dim elements, contiguous in its page).
// Scores are masked per element: key <= query position, and key > position - window
// when a window is set, so the result does not depend on how the tokens were cut
// into steps or tiles.
#include "common.cuh"

namespace axon {

constexpr int FA_BN = 64;       // keys per tile
constexpr int FA_THREADS = 128; // 4 warps
constexpr int FA_MAX_SPLITS = 64;

struct FaParams {
    const __nv_bfloat16* q;      // [tokens][heads * hd]
    const __nv_bfloat16* pool;
    __nv_bfloat16* out;          // [tokens][heads * hd]
    const int32_t* segments;     // [4][n_segments]: slot, q_start, q_len, kv_len
    const int32_t* items;        // [n_items][2]: segment, first token of the tile within the segment
    float* part_o;               // [items][kv_heads][splits][16][hd]   (decode, splits > 1)
    float* part_ml;              // [items][kv_heads][splits][16][2]
    unsigned int* counters;      // [items][kv_heads] arrivals of splits; zero before and after a launch
    PagedKv kv;
    int n_segments, heads, group, tokens_per_tile, n_splits, window;
    float scale_log2;            // scale * log2(e)
    // Decode steps may hand over the q/k/v product itself instead of rotated queries and a written
    // cache (qkv != nullptr): every CTA rotates its own queries, and the CTA whose keys include
    // the new positions rotates and writes their keys and values before it reads them.
    const float* qkv;            // [tokens][qkv_width] float (biases added), or owed the sums in `fold`
    SplitFold fold;
    const float2* table;         // [tokens][hd / 2] (cos, sin), or nullptr: no rotation
    __nv_bfloat16* pool_rw;      // the cache, writable
    int qkv_width, write_kv;
};

// Four consecutive values of the q/k/v product of token t from column col (col % 4 == 0).
__device__ __forceinline__ float4 qkv_at4(const FaParams& p, int t, int col) {
    if (p.fold.partial) return p.fold.at4(t, col);
    return *reinterpret_cast<const float4*>(p.qkv + (long long)t * p.qkv_width + col);
}
// Pairs (i, i + hd/2), i = i0 .. i0 + 3, of one head starting at column `col`, rotated by the
// token's angles (or passed through when there is no table or `rotate` is false).
__device__ __forceinline__ void rotated_quads(const FaParams& p, int t, int col, int half, int i0, bool rotate,
                                              float4& ra, float4& rb) {
    float4 a, b;
    if (p.fold.partial && p.fold.splits <= 8) {
        // both halves' slabs in one batch of loads
        const float4* pa = reinterpret_cast<const float4*>(p.fold.partial + ((long long)((col + i0) >> 7) * p.fold.splits * p.fold.ntok + t) * 128 + ((col + i0) & 127));
        const float4* pb = reinterpret_cast<const float4*>(p.fold.partial + ((long long)((col + half + i0) >> 7) * p.fold.splits * p.fold.ntok + t) * 128 + ((col + half + i0) & 127));
        const long long step = (long long)p.fold.ntok * 32;
        float4 ta[8], tb[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            ta[q] = q < p.fold.splits ? __ldcg(pa + q * step) : make_float4(0.f, 0.f, 0.f, 0.f);
            tb[q] = q < p.fold.splits ? __ldcg(pb + q * step) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        a = make_float4(0.f, 0.f, 0.f, 0.f); b = a;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            a.x += ta[q].x; a.y += ta[q].y; a.z += ta[q].z; a.w += ta[q].w;
            b.x += tb[q].x; b.y += tb[q].y; b.z += tb[q].z; b.w += tb[q].w;
        }
        if (p.fold.bias) {
            const float4 ba = *reinterpret_cast<const float4*>(p.fold.bias + col + i0), bb = *reinterpret_cast<const float4*>(p.fold.bias + col + half + i0);
            a.x += ba.x; a.y += ba.y; a.z += ba.z; a.w += ba.w;
            b.x += bb.x; b.y += bb.y; b.z += bb.z; b.w += bb.w;
        }
    } else {
        a = qkv_at4(p, t, col + i0); b = qkv_at4(p, t, col + half + i0);
    }
    ra = a; rb = b;
    if (rotate && p.table) {
        const float4 c01 = *reinterpret_cast<const float4*>(p.table + (long long)t * half + i0);
        const float4 c23 = *reinterpret_cast<const float4*>(p.table + (long long)t * half + i0 + 2);
        ra.x = a.x * c01.x - b.x * c01.y; rb.x = a.x * c01.y + b.x * c01.x;
        ra.y = a.y * c01.z - b.y * c01.w; rb.y = a.y * c01.w + b.y * c01.z;
        ra.z = a.z * c23.x - b.z * c23.y; rb.z = a.z * c23.y + b.z * c23.x;
        ra.w = a.w * c23.z - b.w * c23.w; rb.w = a.w * c23.w + b.w * c23.z;
    }
}

template <int HD> struct Swz {
    static constexpr int CPR = HD / 8;  // 16-byte chunks per row
    static __device__ __forceinline__ int chunk(int row, int c) {
        if (CPR >= 8) return c ^ (row & 7);
        constexpr int RP = CPR >= 8 ? 1 : 8 / CPR;  // rows per 128 bytes
        return c ^ ((row / RP) % CPR);
    }
    // byte offset of chunk c of row r in a tile
    static __device__ __forceinline__ uint32_t off(int row, int c) { return (uint32_t)(row * CPR + chunk(row, c)) * 16u; }
};

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Gathers 64-key tiles of K and of V for one (request, kv head) into shared memory.  A thread
// copies one 16-byte chunk of every RPP-th row.  When the page size divides 64 a row's page within
// the tile and its place inside that page are the same for every tile, so they are worked out once
// (the division by the page size per row and tile was a third of the decode kernel's instructions).
template <int HD, bool CHECKED> struct KvLoader {
    static constexpr int CPR = HD / 8, RPP = FA_THREADS / CPR, ITER = FA_BN / RPP;
    const int32_t* bt;              // the request's row of the block table
    const __nv_bfloat16* src0;      // this thread's chunk of row 0 of the kv head in page 0 (K plane)
    long long page_stride, v_off;
    unsigned int* fault;            // checked tables (see kv_layout.h): null when off
    int n_pages;
    int ps, pages_per_tile, last_page, kv_len, r0;
    int in_page[ITER], page_of[ITER];
    int ahead[ITER], ahead_tile;    // table entries of tile `ahead_tile`, asked for while the tile before was loaded
    uint32_t dst[ITER];

    __device__ __forceinline__ void init(const __nv_bfloat16* pool, const PagedKv& kv, int slot, int kvh, int kv_len_) {
        const int c = threadIdx.x % CPR;
        r0 = threadIdx.x / CPR;
        ps = kv.page_size; kv_len = kv_len_; fault = kv.fault; n_pages = kv.n_pages;
        bt = kv.block_table + (long long)slot * kv.table_stride;
        src0 = pool + kv.entry_offset + (long long)kvh * ps * HD + c * 8;
        page_stride = kv.page_stride; v_off = kv.v_offset;
        pages_per_tile = FA_BN % ps == 0 ? FA_BN / ps : 0;
        last_page = (kv_len - 1) / ps;
        ahead_tile = -1;
#pragma unroll
        for (int j = 0; j < ITER; ++j) {
            const int r = r0 + RPP * j;
            page_of[j] = r / ps;
            in_page[j] = (r % ps) * HD;
            dst[j] = Swz<HD>::off(r, c);
        }
    }
    __device__ __forceinline__ int checked(int entry) const {
        if ((unsigned)entry > (unsigned)n_pages) { fault[1] = (unsigned)entry; fault[0] = 1u; return n_pages; }
        return entry;
    }
    __device__ __forceinline__ void fetch_entries(int tile) {
        const int first = tile * pages_per_tile;
#pragma unroll
        for (int j = 0; j < ITER; ++j) ahead[j] = bt[min(first + page_of[j], last_page)];
        ahead_tile = tile;
    }
    // rows past the request's length read its last page (fast path) or last position: finite data, masked later
    __device__ __forceinline__ void load(uint32_t k_tile, uint32_t v_tile, int key0) {
        if (pages_per_tile) {
            // Tiles are asked for in ascending order, so the entries of the next one are requested
            // here and are in registers when its turn comes: otherwise every tile's copies wait
            // for a read of the table first.  The tables are complete before the step starts.
            const int tile = key0 / FA_BN;
            if (ahead_tile != tile) fetch_entries(tile);
            // every table entry is loaded before any is checked: a check may store (the fault
            // record), and loads behind a possible store are not issued together
            int page[ITER];
#pragma unroll
            for (int j = 0; j < ITER; ++j) page[j] = ahead[j];
            fetch_entries(tile + 1);
            if (CHECKED) {
#pragma unroll
                for (int j = 0; j < ITER; ++j) page[j] = checked(page[j]);
            }
#pragma unroll
            for (int j = 0; j < ITER; ++j) {
                const __nv_bfloat16* src = src0 + (long long)page[j] * page_stride + in_page[j];
                cp_async16(k_tile + dst[j], src);
                cp_async16(v_tile + dst[j], src + v_off);
            }
        } else {
            int page[ITER];
#pragma unroll
            for (int j = 0; j < ITER; ++j) page[j] = bt[min(key0 + r0 + RPP * j, kv_len - 1) / ps];
            if (CHECKED) {
#pragma unroll
                for (int j = 0; j < ITER; ++j) page[j] = checked(page[j]);
            }
#pragma unroll
            for (int j = 0; j < ITER; ++j) {
                const int pos = min(key0 + r0 + RPP * j, kv_len - 1), lp = pos / ps;
                const __nv_bfloat16* src = src0 + (long long)page[j] * page_stride + (pos - lp * ps) * HD;
                cp_async16(k_tile + dst[j], src);
                cp_async16(v_tile + dst[j], src + v_off);
            }
        }
    }
};
template <int N> __device__ __forceinline__ void cp_async_wait_pending() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// CHECKED: the variant for checked tables (kv_layout.h), a debugging mode.  It is a kernel of its
// own because a check may store: behind a possible store the compiler does not issue the loads
// that follow together, which cost the decode shape 2 us a layer at 7B sizes when the check was
// a run-time branch of the one kernel.
template <int HD, bool DECODE, bool CHECKED>
__global__ void __launch_bounds__(FA_THREADS, (DECODE || HD == 128) ? 2 : 3)   // as many CTAs as shared memory holds
attention_fa_kernel(const FaParams p) {
    constexpr int BM = DECODE ? 16 : 64;
    constexpr int CPR = HD / 8;
    constexpr int KSTEPS = HD / 16;           // k-steps of Q.K^T
    constexpr int NT_S = DECODE ? 2 : 8;      // 8-key score tiles per warp
    constexpr int NT_O = HD / 8;              // 8-dim output tiles
    constexpr int NST = DECODE ? 3 : 2;       // K/V tiles in shared memory: NST - 1 in flight beside the current one
    constexpr uint32_t TILE_BYTES = FA_BN * HD * 2;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    pdl_launch_dependents();
    // The prompt shape waits here: queries and this step's keys come from the kernels before.
    // The decode shape first requests the key tiles that hold only older positions (nothing in
    // this step writes them; lengths and block tables are in place before the step starts), so
    // that the cache streams in while the kernels before are still finishing.
    if (!DECODE) pdl_wait();
    const uint32_t smem = (uint32_t)__cvta_generic_to_shared(smem_raw);
    // decode: [Q | K tiles | V tiles].  prefill: [K tiles | V tiles] with the queries parked in
    // the last V tile until they are in registers (before that tile is first filled)
    const uint32_t k_sm = DECODE ? smem + BM * HD * 2 : smem;
    const uint32_t v_sm = k_sm + NST * TILE_BYTES;
    const uint32_t q_sm = DECODE ? smem : v_sm + (NST - 1) * TILE_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int item = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    // no work list: item i is the whole of segment i (steps of single tokens)
    const int seg = p.items ? p.items[2 * item] : item, tok0 = p.items ? p.items[2 * item + 1] : 0;
    const int slot = p.segments[seg], q_start = p.segments[p.n_segments + seg];
    const int q_len = p.segments[2 * p.n_segments + seg], kv_len = p.segments[3 * p.n_segments + seg];
    const int ntok = min(p.tokens_per_tile, q_len - tok0);
    const int rows_used = ntok * p.group;
    const int pos0 = kv_len - q_len + tok0;           // position of the tile's first token
    const int kv_hi = pos0 + ntok;                    // keys [kv_lo, kv_hi) matter to this tile
    const int kv_lo = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int tile_lo = kv_lo / FA_BN, tile_hi = (kv_hi + FA_BN - 1) / FA_BN;
    const int per = (tile_hi - tile_lo + p.n_splits - 1) / p.n_splits;
    const int t_begin = tile_lo + split * per, t_end = min(tile_hi, t_begin + per);

    const int new_from = kv_len - q_len;              // the segment's first position written by this step
    KvLoader<HD, CHECKED> loader;
    loader.init(p.pool, p.kv, slot, kvh, kv_len);
    if (DECODE) {
#pragma unroll
        for (int st = 0; st < NST - 1; ++st) {
            const int tile = t_begin + st;
            if (tile < t_end && (tile + 1) * FA_BN <= new_from)
                loader.load(k_sm + st * TILE_BYTES, v_sm + st * TILE_BYTES, tile * FA_BN);
            cp_async_commit();
        }
        // (asking for the tiles beyond those into L2 was measured: no gain at batch 8, a loss at 64)
        pdl_wait();
    }
    if (DECODE && p.qkv != nullptr) {
        constexpr int HALF = HD / 2, QUADS = HD / 8;
        const int q_dim = p.heads * HD, kv_dim = p.kv.kv_heads * HD;
        // new keys and values: each by the one CTA whose key tiles hold its position, into the
        // cache (later steps read them there) before that CTA's own loads of those tiles are
        // issued; no other CTA reads that tile
        if (p.write_kv && t_begin < t_end && t_end * FA_BN > pos0) {
            for (int e = threadIdx.x; e < ntok * 2 * QUADS; e += FA_THREADS) {
                const int j = e / (2 * QUADS), is_v = (e / QUADS) & 1, i0 = (e % QUADS) * 4;
                if (pos0 + j < t_begin * FA_BN || pos0 + j >= t_end * FA_BN) continue;
                float4 ra, rb;
                rotated_quads(p, q_start + tok0 + j, q_dim + (is_v ? kv_dim : 0) + kvh * HD, HALF, i0, !is_v, ra, rb);
                __nv_bfloat16* dst = p.pool_rw + (CHECKED ? p.kv.row(slot, pos0 + j, kvh) : p.kv.row_unchecked(slot, pos0 + j, kvh)) +
                                     (is_v ? p.kv.v_offset : 0);
                *reinterpret_cast<uint2*>(dst + i0) = make_uint2(pack_bf16(ra.x, ra.y), pack_bf16(ra.z, ra.w));
                *reinterpret_cast<uint2*>(dst + HALF + i0) = make_uint2(pack_bf16(rb.x, rb.y), pack_bf16(rb.z, rb.w));
            }
            __threadfence();
        }
        // this CTA's queries, rotated, straight into their shared-memory tile
        for (int e = threadIdx.x; e < BM * QUADS; e += FA_THREADS) {
            const int r = e / QUADS, i0 = (e % QUADS) * 4;
            const uint32_t lo = q_sm + Swz<HD>::off(r, i0 >> 3) + (i0 & 4) * 2;
            const uint32_t hi = q_sm + Swz<HD>::off(r, (HALF + i0) >> 3) + ((HALF + i0) & 4) * 2;
            uint2 va = make_uint2(0u, 0u), vb = make_uint2(0u, 0u);
            if (r < rows_used) {
                float4 ra, rb;
                rotated_quads(p, q_start + tok0 + r / p.group, (kvh * p.group + r % p.group) * HD, HALF, i0, true, ra, rb);
                va = make_uint2(pack_bf16(ra.x, ra.y), pack_bf16(ra.z, ra.w));
                vb = make_uint2(pack_bf16(rb.x, rb.y), pack_bf16(rb.z, rb.w));
            }
            asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(lo), "r"(va.x), "r"(va.y) : "memory");
            asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(hi), "r"(vb.x), "r"(vb.y) : "memory");
        }
        __syncthreads();          // the new keys and values are in memory before any thread asks for their tile
    } else
    // ---- Q tile -> shared (rows beyond rows_used are zero)
    for (int e = threadIdx.x; e < BM * CPR; e += FA_THREADS) {
        const int r = e / CPR, c = e % CPR;
        const uint32_t dst = q_sm + Swz<HD>::off(r, c);
        if (r < rows_used) {
            const int tok = q_start + tok0 + r / p.group, head = kvh * p.group + r % p.group;
            cp_async16(dst, p.q + ((long long)tok * p.heads + head) * HD + c * 8);
        } else {
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u));
        }
    }
    if (DECODE) {
        // the tiles of the first NST - 1 that hold new positions, in one group with the queries
        // (the first round waits for every group)
#pragma unroll
        for (int st = 0; st < NST - 1; ++st) {
            const int tile = t_begin + st;
            if (tile < t_end && (tile + 1) * FA_BN > new_from)
                loader.load(k_sm + st * TILE_BYTES, v_sm + st * TILE_BYTES, tile * FA_BN);
        }
        cp_async_commit();
    } else {
        // tiles t_begin .. t_begin + NST - 2 start now, one commit group each (the first also holds Q)
#pragma unroll
        for (int st = 0; st < NST - 1; ++st) {
            if (t_begin + st < t_end)
                loader.load(k_sm + st * TILE_BYTES, v_sm + st * TILE_BYTES, (t_begin + st) * FA_BN);
            cp_async_commit();
        }
    }

    // rows this thread holds: r_a = base + g, r_b = base + g + 8
    const int row_base = DECODE ? 0 : warp * 16;
    const int ra = row_base + g, rb = ra + 8;
    const int pos_a = pos0 + ra / p.group, pos_b = pos0 + rb / p.group;   // query positions
    const int lo_a = (p.window > 0) ? pos_a - p.window + 1 : 0, lo_b = (p.window > 0) ? pos_b - p.window + 1 : 0;

    uint32_t qf[KSTEPS][4];
    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    if (!DECODE) {
        // queries to registers now, so that their shared-memory tile can take keys' values
        cp_async_wait_all();
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int r = row_base + (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * ks + (lane >> 4);
            ldsm_x4(q_sm + Swz<HD>::off(r, c), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        __syncthreads();
    }
    for (int tile = t_begin; tile < t_end; ++tile) {
        const int buf = (tile - t_begin) % NST;
        {
            // the tile NST - 1 ahead goes into the buffer that the previous iteration finished with
            const int ahead = tile + NST - 1, abuf = (ahead - t_begin) % NST;
            if (ahead < t_end)
                loader.load(k_sm + abuf * TILE_BYTES, v_sm + abuf * TILE_BYTES, ahead * FA_BN);
            cp_async_commit();
        }
        // this tile's group (and every older one) has landed.  Decode: the prologue made NST
        // groups (the last holds the queries and the early tiles with new positions), so at the
        // first tile only the group just committed may still be on its way
        if (DECODE && tile == t_begin) cp_async_wait_pending<1>();
        else cp_async_wait_pending<NST - 1>();
        __syncthreads();
        if (DECODE && tile == t_begin) {
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                const int r = row_base + (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * ks + (lane >> 4);
                ldsm_x4(q_sm + Swz<HD>::off(r, c), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
            }
        }
        const uint32_t kt = k_sm + buf * TILE_BYTES, vt = v_sm + buf * TILE_BYTES;
        const int key_base = DECODE ? warp * 16 : 0;   // first key (within the tile) of this warp

        // ---- S = Q K^T
        float s[NT_S][4];
#pragma unroll
        for (int j = 0; j < NT_S; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int jp = 0; jp < NT_S / 2; ++jp) {
                const int n = key_base + jp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8, c = 2 * ks + ((lane >> 3) & 1);
                uint32_t b0, b1, b2, b3;
                ldsm_x4(kt + Swz<HD>::off(n, c), b0, b1, b2, b3);
                mma16816(s[2 * jp], qf[ks], b0, b1);
                mma16816(s[2 * jp + 1], qf[ks], b2, b3);
            }
        }
        // ---- mask, scale, online softmax
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
            const int key = tile * FA_BN + key_base + j * 8 + 2 * t;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int kp = key + i;
                const bool ok_a = kp <= pos_a && kp >= lo_a, ok_b = kp <= pos_b && kp >= lo_b;
                s[j][i] = ok_a ? s[j][i] * p.scale_log2 : -INFINITY;
                s[j][2 + i] = ok_b ? s[j][2 + i] * p.scale_log2 : -INFINITY;
                mx_a = fmaxf(mx_a, s[j][i]);
                mx_b = fmaxf(mx_b, s[j][2 + i]);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float use_a = (mn_a == -INFINITY) ? 0.f : mn_a, use_b = (mn_b == -INFINITY) ? 0.f : mn_b;
        const float corr_a = exp2f(m_a - use_a), corr_b = exp2f(m_b - use_b);   // exp2(-inf) = 0 on the first tile
        m_a = mn_a; m_b = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t pf[NT_S / 2][4];
#pragma unroll
        for (int j = 0; j < NT_S; ++j) {
            const float p0 = exp2f(s[j][0] - use_a), p1 = exp2f(s[j][1] - use_a);
            const float p2 = exp2f(s[j][2] - use_b), p3 = exp2f(s[j][3] - use_b);
            sum_a += p0 + p1; sum_b += p2 + p3;
            pf[j / 2][(j & 1) * 2] = pack_bf16(p0, p1);
            pf[j / 2][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l_a = l_a * corr_a + sum_a;
        l_b = l_b * corr_b + sum_b;
#pragma unroll
        for (int j = 0; j < NT_O; ++j) { o[j][0] *= corr_a; o[j][1] *= corr_a; o[j][2] *= corr_b; o[j][3] *= corr_b; }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < NT_S / 2; ++kk) {
#pragma unroll
            for (int jp = 0; jp < NT_O / 2; ++jp) {
                const int krow = key_base + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * jp + (lane >> 4);
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(vt + Swz<HD>::off(krow, c), b0, b1, b2, b3);
                mma16816(o[2 * jp], pf[kk], b0, b1);
                mma16816(o[2 * jp + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();                      // everyone is done with this buffer before it is refilled
    }
    // the row sums live spread over the quad
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    if (!DECODE) {
        // every warp owns its rows: normalise and store
        const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? rb : ra;
            if (r >= rows_used) continue;
            const int tok = q_start + tok0 + r / p.group, head = kvh * p.group + r % p.group;
            __nv_bfloat16* dst = p.out + ((long long)tok * p.heads + head) * HD;
            const float inv = half ? inv_b : inv_a;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                const uint32_t v = pack_bf16(o[j][2 * half] * inv, o[j][2 * half + 1] * inv);
                *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t) = v;
            }
        }
        return;
    }

    // ---- decode: merge the 4 warps (each saw a quarter of every tile's keys)
    cp_async_wait_all();
    __syncthreads();
    constexpr int MS = HD + 8;     // row stride in floats: the 8 rows of a warp's store fall on different banks
    float* mo = reinterpret_cast<float*>(smem_raw + BM * HD * 2);   // [4][16][MS] over the K/V tiles
    float* mml = mo + 4 * 16 * MS;                                   // [4][16][2]
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
        if (g < rows_used)
            *reinterpret_cast<float2*>(mo + (warp * 16 + g) * MS + j * 8 + 2 * t) = make_float2(o[j][0], o[j][1]);
        if (g + 8 < rows_used)
            *reinterpret_cast<float2*>(mo + (warp * 16 + g + 8) * MS + j * 8 + 2 * t) = make_float2(o[j][2], o[j][3]);
    }
    if (t == 0) {
        mml[(warp * 16 + g) * 2] = m_a; mml[(warp * 16 + g) * 2 + 1] = l_a;
        mml[(warp * 16 + g + 8) * 2] = m_b; mml[(warp * 16 + g + 8) * 2 + 1] = l_b;
    }
    __syncthreads();
    {
        // a thread owns one row and every 8th group of 4 columns: the warps' weights once per thread
        const int r = threadIdx.x >> 3, c4 = (threadIdx.x & 7) * 4;
        if (r < rows_used) {
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) m = fmaxf(m, mml[(w * 16 + r) * 2]);
            const float use = (m == -INFINITY) ? 0.f : m;
            float f[4], l = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                f[w] = exp2f(mml[(w * 16 + r) * 2] - use);
                l += mml[(w * 16 + r) * 2 + 1] * f[w];
            }
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const int tok = q_start + tok0 + r / p.group, head = kvh * p.group + r % p.group;
            const long long base = (((long long)item * gridDim.y + kvh) * p.n_splits + split) * 16 + r;
#pragma unroll
            for (int d = c4; d < HD; d += 32) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float4 v = *reinterpret_cast<const float4*>(mo + (w * 16 + r) * MS + d);
                    acc.x += v.x * f[w]; acc.y += v.y * f[w]; acc.z += v.z * f[w]; acc.w += v.w * f[w];
                }
                if (p.n_splits == 1) {
                    *reinterpret_cast<uint2*>(p.out + ((long long)tok * p.heads + head) * HD + d) =
                        make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
                } else {
                    *reinterpret_cast<float4*>(p.part_o + base * HD + d) = acc;
                }
            }
            if (p.n_splits > 1 && c4 == 0) { p.part_ml[base * 2] = m; p.part_ml[base * 2 + 1] = l; }
        }
    }
    if (p.n_splits == 1 || p.counters == nullptr) return;

    // ---- the CTA that arrives last at this (item, kv head) folds the splits in ascending
    // order and writes the output: no second kernel, and the partials are still in L2
    __shared__ unsigned int arrival;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) arrival = atomicAdd(&p.counters[item * gridDim.y + kvh], 1u);
    __syncthreads();
    if (arrival != (unsigned)(p.n_splits - 1)) return;
    __threadfence();
    float* wm = reinterpret_cast<float*>(smem_raw);      // [splits][16] maxima, then weights
    float* wl = wm + FA_MAX_SPLITS * 16;                  // [splits][16] sums
    const long long base0 = ((long long)item * gridDim.y + kvh) * p.n_splits * 16;
    for (int e = threadIdx.x; e < p.n_splits * 16; e += FA_THREADS) {
        wm[e] = __ldcg(p.part_ml + (base0 + e) * 2);
        wl[e] = __ldcg(p.part_ml + (base0 + e) * 2 + 1);
    }
    __syncthreads();
    if (threadIdx.x < rows_used) {
        const int r = threadIdx.x;
        float m = -INFINITY;
        for (int s = 0; s < p.n_splits; ++s) m = fmaxf(m, wm[s * 16 + r]);
        const float use = (m == -INFINITY) ? 0.f : m;
        float l = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float f = exp2f(wm[s * 16 + r] - use);
            l += wl[s * 16 + r] * f;
            wm[s * 16 + r] = f;
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        for (int s = 0; s < p.n_splits; ++s) wm[s * 16 + r] *= inv;
    }
    __syncthreads();
    constexpr int EPT = (16 * HD + FA_THREADS - 1) / FA_THREADS;   // outputs per thread at most
    float accv[EPT];
#pragma unroll
    for (int k = 0; k < EPT; ++k) accv[k] = 0.f;
    for (int s0 = 0; s0 < p.n_splits; s0 += 4) {
        float tv[EPT][4];
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int e = threadIdx.x + k * FA_THREADS, r = e / HD, d = e % HD;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                tv[k][q] = (e < rows_used * HD && s0 + q < p.n_splits)
                               ? __ldcg(p.part_o + (base0 + (s0 + q) * 16 + r) * HD + d) * wm[(s0 + q) * 16 + r] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < EPT; ++k)
#pragma unroll
            for (int q = 0; q < 4; ++q) accv[k] += tv[k][q];
    }
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int e = threadIdx.x + k * FA_THREADS, r = e / HD, d = e % HD;
        if (e >= rows_used * HD) continue;
        const int tok = q_start + tok0 + r / p.group, head = kvh * p.group + r % p.group;
        p.out[((long long)tok * p.heads + head) * HD + d] = __float2bfloat16_rn(accv[k]);
    }
    if (threadIdx.x == 0) p.counters[item * gridDim.y + kvh] = 0u;    // ready for the next launch
}

// Fold the splits of each (item, kv head, row) in ascending order and normalise.  A thread
// owns float4s of the output; the partials of the first eight splits are requested before
// the weights are known, so the kernel pays one round trip to memory (two beyond 8 splits).
constexpr int FA_COMBINE_THREADS = 256;
template <int HD>
__global__ void __launch_bounds__(FA_COMBINE_THREADS) attention_combine_kernel(const FaParams p) {
    constexpr int V = HD / 4;                                            // float4s per row
    constexpr int EPT = (16 * V + FA_COMBINE_THREADS - 1) / FA_COMBINE_THREADS;
    constexpr int S = 8;                                                 // splits per batch of loads
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.x, kvh = blockIdx.y;
    const int seg = p.items ? p.items[2 * item] : item, tok0 = p.items ? p.items[2 * item + 1] : 0;
    const int q_start = p.segments[p.n_segments + seg], q_len = p.segments[2 * p.n_segments + seg];
    const int rows_used = min(p.tokens_per_tile, q_len - tok0) * p.group;
    __shared__ float wm[FA_MAX_SPLITS * 16], wl[FA_MAX_SPLITS * 16];     // maxima (then weights) and sums of (split, row)
    const long long base0 = ((long long)item * gridDim.y + kvh) * p.n_splits * 16;
    const float2* ml = reinterpret_cast<const float2*>(p.part_ml) + base0;
    const float4* po = reinterpret_cast<const float4*>(p.part_o) + base0 * V;   // [(split * 16 + row) * V + d4]
    for (int e = threadIdx.x; e < p.n_splits * 16; e += FA_COMBINE_THREADS) {
        const float2 v = __ldcg(ml + e);
        wm[e] = v.x;
        wl[e] = v.y;
    }
    float4 tv[EPT][S], acc[EPT];
    auto load = [&](int s0) {
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int e = threadIdx.x + k * FA_COMBINE_THREADS;
#pragma unroll
            for (int q = 0; q < S; ++q)
                tv[k][q] = (e < rows_used * V && s0 + q < p.n_splits) ? __ldcg(po + (long long)(s0 + q) * 16 * V + e)
                                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto fold = [&](int s0) {
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int e = threadIdx.x + k * FA_COMBINE_THREADS, r = min(e / V, 15);
#pragma unroll
            for (int q = 0; q < S; ++q) {
                const float w = s0 + q < p.n_splits ? wm[(s0 + q) * 16 + r] : 0.f;
                acc[k].x += tv[k][q].x * w; acc[k].y += tv[k][q].y * w;
                acc[k].z += tv[k][q].z * w; acc[k].w += tv[k][q].w * w;
            }
        }
    };
    load(0);
    __syncthreads();
    if (threadIdx.x < rows_used) {
        const int r = threadIdx.x;
        float m = -INFINITY;
        for (int s = 0; s < p.n_splits; ++s) m = fmaxf(m, wm[s * 16 + r]);
        const float use = (m == -INFINITY) ? 0.f : m;
        float l = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float f = exp2f(wm[s * 16 + r] - use);
            l += wl[s * 16 + r] * f;
            wm[s * 16 + r] = f;
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        for (int s = 0; s < p.n_splits; ++s) wm[s * 16 + r] *= inv;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < EPT; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    fold(0);
    for (int s0 = S; s0 < p.n_splits; s0 += S) {
        load(s0);
        fold(s0);
    }
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int e = threadIdx.x + k * FA_COMBINE_THREADS;
        if (e >= rows_used * V) continue;
        const int r = e / V, d = (e % V) * 4;
        const int tok = q_start + tok0 + r / p.group, head = kvh * p.group + r % p.group;
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc[k].x, acc[k].y), hi = __floats2bfloat162_rn(acc[k].z, acc[k].w);
        *reinterpret_cast<uint2*>(p.out + ((long long)tok * p.heads + head) * HD + d) =
            make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
}

template <int HD, bool DECODE, bool CHECKED>
static int launch_fa(const FaParams& p, int n_items, int kv_heads, cudaStream_t stream) {
    constexpr int BM = DECODE ? 16 : 64;
    constexpr size_t tiles = (DECODE ? (size_t)BM * HD * 2 : 0) + 2 * (DECODE ? 3 : 2) * (size_t)FA_BN * HD * 2;
    constexpr size_t merge = DECODE ? (size_t)BM * HD * 2 + (4 * 16 * (HD + 8) + 4 * 16 * 2) * sizeof(float) : 0;
    constexpr size_t smem = tiles > merge ? tiles : merge;
    if (int st = ensure_dynamic_smem<attention_fa_kernel<HD, DECODE, CHECKED>>(smem, "axon_attention_fa")) return st;
    dim3 grid(n_items, kv_heads, DECODE ? p.n_splits : 1);
    launch_pdl(attention_fa_kernel<HD, DECODE, CHECKED>, grid, dim3(FA_THREADS), smem, stream, p);
    int st = launch_status("axon_attention_fa");
    if (st != AXON_OK) return st;
    if (DECODE && p.n_splits > 1 && p.counters == nullptr) {
        launch_pdl(attention_combine_kernel<HD>, dim3(n_items, kv_heads), dim3(FA_COMBINE_THREADS), 0, stream, p);
        st = launch_status("axon_attention_fa combine");
    }
    return st;
}

}  // namespace axon

using namespace axon;

// How many floats of scratch a decode launch with these sizes needs (0 when splits == 1).
AXON_API long long axon_attention_fa_scratch_floats(int n_items, int kv_heads, int n_splits, int head_dim) {
    if (n_splits <= 1) return 0;
    return (long long)n_items * kv_heads * n_splits * 16 * (head_dim + 2);
}

// decode != 0: tiles of 16 rows with `n_splits` key shares; else tiles of 64 rows.
// `counters` (may be null): n_items * kv_heads zeroed 32-bit counters, left zeroed; with them
// the split that finishes last folds the partials itself, without them a second kernel does.
// tokens_per_tile * group rows must fit the tile.  scratch: see above (may be null when
// n_splits == 1).  Head sizes 16, 32, 64, 128; group <= 16 (decode) or 64 (prefill).
namespace {
struct FusedQkv {            // see FaParams::qkv
    const float* qkv = nullptr;
    SplitFold fold{nullptr, nullptr, 0, 0};
    const float2* table = nullptr;
    int qkv_width = 0, write_kv = 0;
};
}

static int attention_fa_launch(const void* q, const void* pool, void* out, const int32_t* segments, int n_segments,
                               const int32_t* items, int n_items, const AxonKvLayout* layout, int heads,
                               float scale, int window, int decode, int tokens_per_tile, int n_splits,
                               float* scratch, unsigned int* counters, const FusedQkv& fused, cudaStream_t stream) {
    if (n_items <= 0) return AXON_OK;
    const int hd = layout->head_dim, kvh = layout->kv_heads;
    if (heads % kvh) { set_error("axon_attention_fa: %d heads over %d kv heads", heads, kvh); return AXON_BAD_ARGUMENT; }
    const int group = heads / kvh, bm = decode ? 16 : 64;
    if (tokens_per_tile < 1 || tokens_per_tile * group > bm) { set_error("axon_attention_fa: %d tokens x %d heads do not fit a tile of %d rows", tokens_per_tile, group, bm); return AXON_BAD_ARGUMENT; }
    if (n_splits < 1 || n_splits > FA_MAX_SPLITS || (!decode && n_splits != 1)) { set_error("axon_attention_fa: bad split count %d (1..%d; 1 for prefill tiles)", n_splits, FA_MAX_SPLITS); return AXON_BAD_ARGUMENT; }
    if (n_splits > 1 && scratch == nullptr) { set_error("axon_attention_fa: %d key splits need scratch memory for their partial results", n_splits); return AXON_BAD_ARGUMENT; }
    if (layout->planes == 1 || (layout->v_dim > 0 && layout->v_dim != hd)) { set_error("axon_attention_fa: takes caches with key and value planes of one width"); return AXON_BAD_ARGUMENT; }
    if (((uintptr_t)q | (uintptr_t)pool | (uintptr_t)out) & 15) { set_error("axon_attention_fa: operands must be 16-byte aligned"); return AXON_BAD_ARGUMENT; }
    FaParams p;
    p.q = (const __nv_bfloat16*)q; p.pool = (const __nv_bfloat16*)pool; p.out = (__nv_bfloat16*)out;
    p.segments = segments; p.items = items;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (long long)n_items * kvh * n_splits * 16 * hd : nullptr;
    p.counters = (n_splits > 1 && scratch) ? counters : nullptr;
    p.kv = to_paged(layout);
    p.n_segments = n_segments; p.heads = heads; p.group = group; p.tokens_per_tile = tokens_per_tile;
    p.n_splits = n_splits; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.qkv = fused.qkv; p.fold = fused.fold; p.table = fused.table; p.pool_rw = (__nv_bfloat16*)const_cast<void*>(pool);
    p.qkv_width = fused.qkv_width; p.write_kv = fused.write_kv;
#define AXON_FA_CASE(HD)                                                                         \
    case HD:                                                                                     \
        if (p.kv.fault != nullptr)                                                               \
            return decode ? launch_fa<HD, true, true>(p, n_items, kvh, stream) : launch_fa<HD, false, true>(p, n_items, kvh, stream); \
        return decode ? launch_fa<HD, true, false>(p, n_items, kvh, stream) : launch_fa<HD, false, false>(p, n_items, kvh, stream);
    switch (hd) {
        AXON_FA_CASE(16)
        AXON_FA_CASE(32)
        AXON_FA_CASE(64)
        AXON_FA_CASE(128)
        default: set_error("axon_attention_fa: head size %d is not 16, 32, 64 or 128", hd); return AXON_BAD_ARGUMENT;
    }
#undef AXON_FA_CASE
}

AXON_API int axon_attention_fa(const void* q, const void* pool, void* out, const int32_t* segments, int n_segments,
                               const int32_t* items, int n_items, const AxonKvLayout* layout, int heads,
                               float scale, int window, int decode, int tokens_per_tile, int n_splits,
                               float* scratch, unsigned int* counters, cudaStream_t stream) {
    return attention_fa_launch(q, pool, out, segments, n_segments, items, n_items, layout, heads, scale, window, decode,
                               tokens_per_tile, n_splits, scratch, counters, FusedQkv{}, stream);
}

// Decode steps (segment i is item i, and no segment holds more than `max_q_len` tokens, which
// must not exceed `tokens_per_tile`: a longer segment would lose its further tokens, so the call
// is refused): rotation, cache write and attention in one kernel.  Each new key and value is
// written by the CTA whose share of the key tiles holds its position, before that CTA loads the tile.  qkv: float [tokens][(heads + 2 kv_heads) * hd] with
// biases added, or (partial != null) still owed the partial sums of a deferred split-K product
// with its bias.  table: (cos, sin) [tokens][hd / 2] for pairs (i, i + hd / 2) over the whole
// head, or null for no rotation.  write_kv == 0: the cache holds the new positions already
// (a layer reading another layer's cache).  Otherwise as axon_attention_fa with decode != 0.
AXON_API int axon_attention_fa_decode_fused(const float* qkv, const float* partial, int fold_splits, int fold_ntok,
                                            const float* bias, const float* table, int write_kv, void* pool, void* out,
                                            const int32_t* segments, int n_segments, const AxonKvLayout* layout,
                                            int heads, float scale, int window, int tokens_per_tile, int max_q_len,
                                            int n_splits, float* scratch, unsigned int* counters, cudaStream_t stream) {
    const int hd = layout->head_dim;
    if (max_q_len < 1 || max_q_len > tokens_per_tile) { set_error("axon_attention_fa_decode_fused: segments of up to %d tokens do not fit tiles of %d", max_q_len, tokens_per_tile); return AXON_BAD_ARGUMENT; }
    if (qkv == nullptr) { set_error("axon_attention_fa_decode_fused: no q/k/v product given"); return AXON_BAD_ARGUMENT; }
    if (hd % 8) { set_error("axon_attention_fa_decode_fused: head size %d is not a multiple of 8", hd); return AXON_BAD_ARGUMENT; }
    if (partial != nullptr && (fold_splits < 1 || fold_ntok < 1)) { set_error("axon_attention_fa_decode_fused: bad partial sums"); return AXON_BAD_ARGUMENT; }
    if (((uintptr_t)qkv | (uintptr_t)partial | (uintptr_t)bias | (uintptr_t)table) & 15) { set_error("axon_attention_fa_decode_fused: operands must be 16-byte aligned"); return AXON_BAD_ARGUMENT; }
    if ((layout->page_stride * 2) % 16 || (layout->entry_offset * 2) % 16 || (layout->v_offset * 2) % 16) { set_error("axon_attention_fa_decode_fused: cache planes must be 16-byte aligned"); return AXON_BAD_ARGUMENT; }
    FusedQkv f;
    f.qkv = qkv;
    f.fold = SplitFold{partial, partial ? bias : nullptr, fold_splits, fold_ntok};
    f.table = (const float2*)table;
    f.qkv_width = (heads + 2 * layout->kv_heads) * hd;
    f.write_kv = write_kv;
    return attention_fa_launch(qkv, pool, out, segments, n_segments, nullptr, n_segments, layout, heads, scale, window, 1,
                               tokens_per_tile, n_splits, scratch, counters, f, stream);
}

// ---------------------------------------------------------------------------
// The variant for callers that cannot allocate: see attention_fa_noalloc.h.
#include "attention_fa_noalloc.h"

// The split partials of one launch.  In host code this name is only a stand-in for
// the symbol, not a device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_fa_noalloc_scratch[AXON_FA_NOALLOC_SCRATCH_FLOATS];
// Arrival counters of the splits (zero at load, and every launch leaves them zero).
static __device__ __align__(256) unsigned int g_fa_noalloc_counters[AXON_FA_NOALLOC_COUNTERS];

namespace {
constexpr int kMaxDevices = 64;
float* g_fa_noalloc_ptr[kMaxDevices] = {};   // device address of the array, per device, once looked up
unsigned int* g_fa_noalloc_counters_ptr[kMaxDevices] = {};
}

int axon_attention_fa_decode_noalloc(const void* q, const void* pool, void* out, const int32_t* segments,
                                     int n_segments, const int32_t* items, int n_items,
                                     const AxonKvLayout* layout, int heads, float scale, int window,
                                     int tokens_per_tile, int n_splits, cudaStream_t stream) {
    if (n_items <= 0) return AXON_OK;
    if (layout == nullptr || n_splits < 1) { set_error("axon_attention_fa_decode_noalloc: bad arguments"); return AXON_BAD_ARGUMENT; }
    const long long need = (long long)n_items * layout->kv_heads * n_splits * 16 * (layout->head_dim + 2);
    if (need > AXON_FA_NOALLOC_SCRATCH_FLOATS) {
        set_error("axon_attention_fa_decode_noalloc: %d items x %d kv heads x %d splits need %lld floats of scratch; "
                  "the built-in array holds %lld (use fewer splits, or axon_attention_fa with your own scratch)",
                  n_items, layout->kv_heads, n_splits, need, (long long)AXON_FA_NOALLOC_SCRATCH_FLOATS);
        return AXON_BAD_ARGUMENT;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("axon_attention_fa_decode_noalloc: cudaGetDevice: %s", e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
        return AXON_CUDA_ERROR;
    }
    if (g_fa_noalloc_ptr[dev] == nullptr) {
        // set-up, once per device, with that device current
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_fa_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("axon_attention_fa_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return AXON_CUDA_ERROR;
        }
        unsigned int* cptr = nullptr;
        e = cudaGetSymbolAddress((void**)&cptr, g_fa_noalloc_counters);
        if (e != cudaSuccess || cptr == nullptr) {
            set_error("axon_attention_fa_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return AXON_CUDA_ERROR;
        }
        g_fa_noalloc_counters_ptr[dev] = cptr;
        g_fa_noalloc_ptr[dev] = ptr;
    }
    return axon_attention_fa(q, pool, out, segments, n_segments, items, n_items, layout, heads, scale, window,
                             /*decode=*/1, tokens_per_tile, n_splits, g_fa_noalloc_ptr[dev],
                             (long long)n_items * layout->kv_heads <= AXON_FA_NOALLOC_COUNTERS ? g_fa_noalloc_counters_ptr[dev] : nullptr,
                             stream);
}
