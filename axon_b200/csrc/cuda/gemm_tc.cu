// bfloat16 products on the 5th-generation tensor cores: out[m][n] = sum_k a[m][k] w[n][k].
//
// One CTA computes a 128 x BN tile of the output (BN = 256 or 128).  Operands are both
// K-major, so activations [M][K] and weights [N][K] are loaded as they lie in memory:
// a TMA producer thread copies 128 x 64 and BN x 64 element boxes (128-byte swizzle)
// into a ring of shared-memory stages; one MMA thread issues tcgen05.mma (M 128, N BN,
// K 16) four times per stage into a float accumulator in tensor memory and releases the
// stage with tcgen05.commit; eight epilogue warps read the accumulator back with
// tcgen05.ld (a thread per output row, two warps per 32 rows sharing the columns) and apply
// the epilogue: store as float or bfloat16 with an optional bias, add into a float residual,
// or SwiGLU over interleaved gate/up columns.  A warp stages its 32 rows x 32 columns in
// shared memory (the ring is free by then) and hands them to TMA: a thread per row writing
// straight to global memory touches 32 rows per store instruction, which made the epilogue
// as long as half the K loop.  The residual is added by the TMA reduce (one add per element,
// so the order is fixed).  Tails in M, N and K are zero-filled by TMA on the way in and
// clipped on the way out; outputs that TMA cannot address (rows not 16-byte multiples) take
// the stores from registers.
//
// Every wait on an mbarrier is bounded: when a wait gives up, the kernel records it in a
// device flag (read with axon_gemm_tc_status) and carries on to its end, so tensor
// memory is always freed and nothing spins forever.
#include "tcgen05.cuh"

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace axon {

constexpr int TC_BM = 128, TC_BK = 64;
enum { TC_STORE_F32 = 0, TC_STORE_BF16 = 1, TC_RESIDUAL = 2, TC_SWIGLU = 3 };

// RM: 128-row sub-tiles of activations per CTA (1 or 2).  With two, both MMAs of a k-step
// read the same weight tile from shared memory, so a CTA needs 1.5x fewer operand bytes per
// FLOP; the operand feed from L2, not the tensor pipe, bounds this kernel at prefill sizes.
// BN: any multiple of 32 up to 256; RM * BN float columns of tensor memory hold the tile.
constexpr int TC_THREADS = 320;      // TMA warp, MMA warp, eight epilogue warps

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t smem, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t smem, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int BN, int STAGES, int EPI, int RM, bool TMA_OUT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out,
               const float* __restrict__ bias, void* __restrict__ out, int M, int N, int K, int ldo, int m_tiles,
               uint32_t stuck_wait_limit) {
    // stuck_wait_limit != 0 (tests of the failure path only): the MMA thread never tells the
    // epilogue that the accumulator is complete, and the epilogue's wait gives up after that many
    // polls.  The kernel must then still end in order: error flag set, tensor memory freed.
    constexpr uint32_t A_BYTES = RM * TC_BM * TC_BK * 2, W_BYTES = BN * TC_BK * 2, STAGE_BYTES = A_BYTES + W_BYTES;
    constexpr uint32_t TMEM_COLS = RM * BN <= 32 ? 32 : RM * BN <= 64 ? 64 : RM * BN <= 128 ? 128 : RM * BN <= 256 ? 256 : 512;
    extern __shared__ unsigned char smem_dyn[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2];
    __shared__ uint32_t tmem_slot;
    const uint32_t full0 = (uint32_t)__cvta_generic_to_shared(&bars[0]);
    const uint32_t empty0 = full0 + 8 * STAGES, tmem_full = full0 + 16 * STAGES, mma_done = tmem_full + 8;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tile = blockIdx.x % m_tiles, n_tile = blockIdx.x / m_tiles;
    const int m0 = m_tile * TC_BM * RM, n0 = n_tile * BN;
    const int k_stages = (K + TC_BK - 1) / TC_BK;
    // the kernel after this one may begin its own set-up; this one fills its ring with weights
    // and waits for the kernels before it only where it first needs the activations
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tmem_full, 1);
        mbar_init(mma_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // this warp owns tensor memory: RM * BN float columns for the accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = tmem_slot;

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            const int early = k_stages < STAGES ? k_stages : STAGES;
            for (int ks = 0; ks < early; ++ks) {           // weights: nothing in a step writes them
                mbar_expect_tx(full0 + 8 * ks, STAGE_BYTES);
                tma_load_2d(smem_base + ks * STAGE_BYTES + A_BYTES, &map_w, ks * TC_BK, n0, full0 + 8 * ks);
            }
            pdl_wait();
            for (int ks = 0; ks < early; ++ks)
                tma_load_2d(smem_base + ks * STAGE_BYTES, &map_a, ks * TC_BK, m0, full0 + 8 * ks);
            for (int ks = early; ks < k_stages; ++ks) {
                const int s = ks % STAGES;
                mbar_wait(empty0 + 8 * s, ((ks / STAGES) - 1) & 1, 0);
                const uint32_t sa = smem_base + s * STAGE_BYTES, sw = sa + A_BYTES;
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_2d(sa, &map_a, ks * TC_BK, m0, full0 + 8 * s);
                tma_load_2d(sw, &map_w, ks * TC_BK, n0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(TC_BM, BN);
            for (int ks = 0; ks < k_stages; ++ks) {
                const int s = ks % STAGES;
                mbar_wait(full0 + 8 * s, (ks / STAGES) & 1, 1);
                tc_fence_after();
                const uint32_t sa = smem_base + s * STAGE_BYTES, sw = sa + A_BYTES;
                const uint64_t da = smem_desc(sa), db = smem_desc(sw);
#pragma unroll
                for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
                    // 16 elements = 32 bytes along K inside the swizzled row: +2 in the address field;
                    // sub-tile rm of the activations lies 16 KiB (+1024) further, its accumulator BN columns further
#pragma unroll
                    for (int rm = 0; rm < RM; ++rm)
                        umma(tmem_acc + (uint32_t)(rm * BN), da + (uint64_t)(rm * 1024 + 2 * k), db + (uint64_t)(2 * k),
                             idesc, (ks | k) ? 1u : 0u);
                }
                umma_commit(empty0 + 8 * s);      // the stage is free once these MMAs have read it
            }
            if (stuck_wait_limit == 0) {
                umma_commit(tmem_full);           // the accumulator is complete
            } else {
                // the failure test: the epilogue is never told; this thread still sees the MMAs
                // through, so that nothing is in flight when tensor memory is freed
                umma_commit(mma_done);
                mbar_wait(mma_done, 0, 1);
            }
        }
    } else {
        // ---- epilogue: warps 2..9; a warp reads tensor-memory lanes 32 * (warp % 4) .., and the
        // two warps of a lane quarter take every other 32-column chunk
        mbar_wait(tmem_full, 0, 2, stuck_wait_limit ? stuck_wait_limit : TC_WAIT_LIMIT);
        __syncwarp();
        tc_fence_after();
        pdl_wait();          // before the output is read or written (the producer passed this long ago)
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const uint32_t lane_addr = tmem_acc + ((uint32_t)(quarter * 32) << 16);
        if constexpr (TMA_OUT) {
            // every MMA has read the ring and every load has landed: the ring is scratch now.
            // Two 4 KiB buffers per warp: a chunk is staged while the one before is still being read out.
            const uint32_t stage = smem_base + (uint32_t)(warp - 2) * 8192u;
            int iter = 0;
#pragma unroll 1
            for (int cc = half; cc < RM * (BN / 32); cc += 2) {
                const int rm = cc / (BN / 32), c = cc % (BN / 32);
                const int row0 = m0 + rm * TC_BM + quarter * 32, nc = n0 + c * 32;
                if (row0 >= M || nc >= N) continue;               // the same for the whole warp
                const uint32_t buf = stage + (uint32_t)(iter & 1) * 4096u;
                if (iter >= 2) {
                    if (lane == 0) bulk_wait_read<1>();           // the store that read this buffer is done with it
                    __syncwarp();
                }
                uint32_t r[32];
                tmem_ld32(lane_addr + (uint32_t)(rm * BN + c * 32), r);
                if (bias) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (nc + i < N) r[i] = __float_as_uint(__uint_as_float(r[i]) + bias[nc + i]);
                }
                if (EPI == TC_SWIGLU) {
                    // 16 outputs = 32 bytes per row; 32-byte swizzle: chunk bit 0 ^= row bit 2
                    uint32_t pk[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float g0 = __uint_as_float(r[4 * i]), u0 = __uint_as_float(r[4 * i + 1]);
                        const float g1 = __uint_as_float(r[4 * i + 2]), u1 = __uint_as_float(r[4 * i + 3]);
                        pk[i] = pack_bf16(__fdividef(g0, 1.0f + __expf(-g0)) * u0, __fdividef(g1, 1.0f + __expf(-g1)) * u1);
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        st_shared_v4(buf + lane * 32 + ((j ^ ((lane >> 2) & 1)) << 4), pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                } else if (EPI == TC_STORE_BF16) {
                    // 32 outputs = 64 bytes per row; 64-byte swizzle: chunk bits 0..1 ^= row bits 1..2
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        st_shared_v4(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4),
                                     pack_bf16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                                     pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                                     pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                                     pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
                } else {
                    // 32 floats = 128 bytes per row; 128-byte swizzle
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        st_shared_v4(buf + sw128_offset(lane, j), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    const int x = EPI == TC_SWIGLU ? (nc >> 1) : nc;
                    if (EPI == TC_RESIDUAL) tma_reduce_add_2d(&map_out, buf, x, row0);
                    else tma_store_2d(&map_out, buf, x, row0);
                    bulk_commit();
                }
                ++iter;
            }
            if (lane == 0) bulk_wait_read<0>();                   // shared memory must outlive the reads
        } else {
#pragma unroll 1
        for (int cc = half; cc < RM * (BN / 32); cc += 2) {
            const int rm = cc / (BN / 32), c = cc % (BN / 32);
            const int m = m0 + rm * TC_BM + quarter * 32 + lane;
            uint32_t r[32];
            tmem_ld32(lane_addr + (uint32_t)(rm * BN + c * 32), r);
            const int nc = n0 + c * 32;
            if (m >= M || nc >= N) continue;
            if (EPI == TC_SWIGLU) {
                __nv_bfloat16* dst = (__nv_bfloat16*)out + (long long)m * ldo + (nc >> 1);
                float res[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float gv = __uint_as_float(r[2 * i]), uv = __uint_as_float(r[2 * i + 1]);
                    if (bias && nc + 2 * i + 1 < N) { gv += bias[nc + 2 * i]; uv += bias[nc + 2 * i + 1]; }
                    res[i] = gv / (1.0f + __expf(-gv)) * uv;
                }
                if (nc + 32 <= N && ((((uintptr_t)dst) & 15) == 0)) {
                    uint32_t pk[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        __nv_bfloat162 v = __floats2bfloat162_rn(res[2 * i], res[2 * i + 1]);
                        pk[i] = *reinterpret_cast<uint32_t*>(&v);
                    }
                    *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *reinterpret_cast<uint4*>(dst + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (nc + 2 * i + 1 < N) dst[i] = __float2bfloat16_rn(res[i]);
                }
            } else if (EPI == TC_STORE_BF16) {
                __nv_bfloat16* dst = (__nv_bfloat16*)out + (long long)m * ldo + nc;
                const bool full = (nc + 32 <= N) && ((((uintptr_t)dst) & 15) == 0);
                if (full) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t pk[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float a = __uint_as_float(r[8 * i + 2 * j]), b = __uint_as_float(r[8 * i + 2 * j + 1]);
                            if (bias) { a += bias[nc + 8 * i + 2 * j]; b += bias[nc + 8 * i + 2 * j + 1]; }
                            __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
                            pk[j] = *reinterpret_cast<uint32_t*>(&v);
                        }
                        *reinterpret_cast<uint4*>(dst + 8 * i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (nc + i < N) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]) + (bias ? bias[nc + i] : 0.f));
                }
            } else {
                float* dst = (float*)out + (long long)m * ldo + nc;
                const bool full = (nc + 32 <= N) && ((((uintptr_t)dst) & 15) == 0);
                if (full) {
                    // what the residual epilogue adds to is loaded before any store of the chunk,
                    // so that the eight loads are in flight together
                    float4 o[8];
                    if (EPI == TC_RESIDUAL) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = *reinterpret_cast<const float4*>(dst + 4 * i);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                               __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                        if (bias) { v.x += bias[nc + 4 * i]; v.y += bias[nc + 4 * i + 1]; v.z += bias[nc + 4 * i + 2]; v.w += bias[nc + 4 * i + 3]; }
                        if (EPI == TC_RESIDUAL) { v.x += o[i].x; v.y += o[i].y; v.z += o[i].z; v.w += o[i].w; }
                        *reinterpret_cast<float4*>(dst + 4 * i) = v;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (nc + i < N) {
                            float v = __uint_as_float(r[i]) + (bias ? bias[nc + i] : 0.f);
                            if (EPI == TC_RESIDUAL) v += dst[i];
                            dst[i] = v;
                        }
                    }
                }
            }
        }
        }   // !TMA_OUT
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Few activation rows (decode): the operands swap roles.  The weights are the 128-row
// operand of the MMA and the tokens (padded to NTOK = 16, 32 or 64) its columns, so a
// CTA streams a 128-row slab of weights through TMA at full width whatever the batch
// size; the product is bound by reading the weights once from HBM.  To fill the machine
// when a matrix has few 128-row tiles, K is cut into `splits` slabs, one CTA each: every
// CTA writes its partial tile to scratch, and the CTA that arrives last at the tile's
// counter adds the partials in slab order (so the sum does not depend on timing) and
// applies the epilogue.  Without counters the partial tiles are the result: the kernel
// that reads the output next (a norm, the rotation) adds them on its way (SplitFold), which
// takes the fence, the counter and the gathering pass off this kernel's tail.  In tensor memory a lane is a weight row and a column a token,
// so for a fixed token the 32 lanes of a warp write 32 consecutive outputs.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// What the residual epilogue adds to: loaded ahead of the stores, many at a time, because
// a load behind a store to the same array cannot be moved up by the compiler and a chain
// of dependent global loads is what small kernels spend their time on.
template <int EPI>
__device__ __forceinline__ float swap_old(int row, int tok, int N, const void* out, int ldo) {
    if (EPI != TC_RESIDUAL || row >= N) return 0.f;
    return ((const float*)out)[(long long)tok * ldo + row];
}

template <int EPI>
__device__ __forceinline__ void swap_store(float v, float old, int row, int tok, int N, const float* bias, void* out,
                                           int ldo) {
    // v is the product for (weight row, token); all 32 lanes hold consecutive rows
    if (EPI == TC_SWIGLU) {
        if (bias && row < N) v += bias[row];
        const float other = __shfl_xor_sync(0xffffffffu, v, 1);      // row ^ 1: the up value of a gate row
        if (!(row & 1) && row + 1 < N) {
            const float r = v / (1.0f + __expf(-v)) * other;
            ((__nv_bfloat16*)out)[(long long)tok * ldo + (row >> 1)] = __float2bfloat16_rn(r);
        }
        return;
    }
    if (row >= N) return;
    if (bias) v += bias[row];
    const long long o = (long long)tok * ldo + row;
    if (EPI == TC_STORE_F32) ((float*)out)[o] = v;
    else if (EPI == TC_STORE_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v);
    else ((float*)out)[o] = old + v;
}

// R: 128-row sub-tiles per CTA (1 or 2).  Two halve the number of CTAs of a matrix with
// many rows, so that one CTA per SM covers it and the next kernel's CTAs fit beside it
// to preload their weights; splitting K is for R == 1 only.
template <int NTOK, int STAGES, int EPI, int R>
__global__ void __launch_bounds__(192)
gemm_tc_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const float* __restrict__ bias, void* out, float* __restrict__ partial,
                    unsigned int* __restrict__ counters, int M, int N, int K, int ldo, int splits, int per_split) {
    constexpr uint32_t W_BYTES = R * 128 * TC_BK * 2, X_BYTES = NTOK * TC_BK * 2, STAGE_BYTES = W_BYTES + X_BYTES;
    constexpr uint32_t TMEM_COLS = R * NTOK < 32 ? 32 : R * NTOK;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t smem_base = ((uint32_t)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ unsigned int arrival;
    const uint32_t full0 = (uint32_t)__cvta_generic_to_shared(&bars[0]);
    const uint32_t empty0 = full0 + 8 * STAGES, tmem_full = full0 + 16 * STAGES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / splits, split = blockIdx.x % splits;
    const int n0 = tile * 128 * R;
    // more than NTOK tokens: blockIdx.y picks the block of NTOK; M_all tokens in all, Mb in this block
    const int t0 = blockIdx.y * NTOK, M_all = M, m_pad = gridDim.y * NTOK;
    M = min(NTOK, M_all - t0);
    out = EPI == TC_STORE_BF16 || EPI == TC_SWIGLU ? (void*)((__nv_bfloat16*)out + (long long)t0 * ldo)
                                                   : (void*)((float*)out + (long long)t0 * ldo);
    const int k_total = (K + TC_BK - 1) / TC_BK;
    const int ks_begin = split * per_split, ks_end = min(k_total, ks_begin + per_split);
    const int k_stages = ks_end - ks_begin;          // >= 1 by construction of `splits`
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
            // the weights do not depend on the kernel before this one: start streaming them
            // into every stage, and wait for that kernel only before the activations
            const int ahead = k_stages < STAGES ? k_stages : STAGES;
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(full0 + 8 * i, STAGE_BYTES);
                tma_load_2d(smem_base + i * STAGE_BYTES, &map_w, (ks_begin + i) * TC_BK, n0, full0 + 8 * i);
            }
            // (asking for further boxes into L2 here was measured: it slows the step down, the more
            // boxes the more, because the requests queue ahead of the loads that follow)
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(smem_base + i * STAGE_BYTES + W_BYTES, &map_x, (ks_begin + i) * TC_BK, t0, full0 + 8 * i);
            for (int i = ahead; i < k_stages; ++i) {
                const int s = i % STAGES;
                mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, 0);
                const uint32_t sw = smem_base + s * STAGE_BYTES, sx = sw + W_BYTES;
                mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_2d(sw, &map_w, (ks_begin + i) * TC_BK, n0, full0 + 8 * s);
                tma_load_2d(sx, &map_x, (ks_begin + i) * TC_BK, t0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(128, NTOK);
            for (int i = 0; i < k_stages; ++i) {
                const int s = i % STAGES;
                mbar_wait(full0 + 8 * s, (i / STAGES) & 1, 1);
                tc_fence_after();
                const uint32_t sw = smem_base + s * STAGE_BYTES, sx = sw + W_BYTES;
                const uint64_t da = smem_desc(sw), db = smem_desc(sx);
#pragma unroll
                for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)
#pragma unroll
                    for (int r = 0; r < R; ++r)   // sub-tile r: 128 rows further (16 KiB), NTOK columns further
                        umma(tmem_acc + (uint32_t)(r * NTOK), da + (uint64_t)(r * 1024 + 2 * k), db + (uint64_t)(2 * k),
                             idesc, (i | k) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);
            }
            umma_commit(tmem_full);
        }
    } else {
        pdl_wait();                                                // before anything is written
        mbar_wait(tmem_full, 0, 2);
        tc_fence_after();
        const int quarter = warp & 3;
        const uint32_t lane_addr = tmem_acc + ((uint32_t)(quarter * 32) << 16);
        if (R > 1) {
            // whole-K sub-tiles, one after the other
#pragma unroll 1
            for (int r = 0; r < R; ++r) {
                const int row_r = n0 + r * 128 + quarter * 32 + lane;
#pragma unroll
                for (int c = 0; c < NTOK / 16; ++c) {
                    uint32_t v[16];
                    float old[16];
                    tmem_ld16(lane_addr + (uint32_t)(r * NTOK + c * 16), v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) old[i] = (c * 16 + i < M) ? swap_old<EPI>(row_r, c * 16 + i, N, out, ldo) : 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (c * 16 + i < M) swap_store<EPI>(__uint_as_float(v[i]), old[i], row_r, c * 16 + i, N, bias, out, ldo);
                }
            }
            tc_fence_before();
        } else {
        const int row = n0 + quarter * 32 + lane;                  // this lane's weight row
        if (splits == 1) {
            // sixteen tokens at a time: tensor memory -> epilogue -> memory
#pragma unroll 1
            for (int c = 0; c < NTOK / 16 && c * 16 < M; ++c) {
                uint32_t r[16];
                float old[16];
                tmem_ld16(lane_addr + (uint32_t)(c * 16), r);
#pragma unroll
                for (int i = 0; i < 16; ++i) old[i] = (c * 16 + i < M) ? swap_old<EPI>(row, c * 16 + i, N, out, ldo) : 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (c * 16 + i < M) swap_store<EPI>(__uint_as_float(r[i]), old[i], row, c * 16 + i, N, bias, out, ldo);
            }
            tc_fence_before();
        } else {
            // partial[tile][split][token][row of this tile]; then the last CTA of the tile folds
            // (or, without counters, the reader of the output does)
            float* mine = partial + ((long long)(tile * splits + split) * m_pad + t0) * 128 + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < NTOK / 16 && c * 16 < M; ++c) {
                uint32_t r[16];
                tmem_ld16(lane_addr + (uint32_t)(c * 16), r);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (c * 16 + i < M) mine[(c * 16 + i) * 128] = __uint_as_float(r[i]);
            }
            tc_fence_before();
            if (counters != nullptr) {
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");             // the four epilogue warps
            if (threadIdx.x == 64) arrival = atomicAdd(&counters[tile * gridDim.y + blockIdx.y], 1u);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (arrival == (unsigned)(splits - 1)) {
                __threadfence();
                const float* all = partial + ((long long)tile * splits * m_pad + t0) * 128 + quarter * 32 + lane;
                // G tokens and four slabs at a time: up to 64 independent loads in flight per
                // thread, summed in slab order (adding the zeros of absent slabs changes nothing)
                constexpr int G = NTOK >= 32 ? 16 : 8;
#pragma unroll 1
                for (int j0 = 0; j0 < M; j0 += G) {
                    float v[G], old[G];
#pragma unroll
                    for (int u = 0; u < G; ++u) {
                        v[u] = 0.f;
                        old[u] = (j0 + u < M) ? swap_old<EPI>(row, j0 + u, N, out, ldo) : 0.f;
                    }
#pragma unroll 1
                    for (int s0 = 0; s0 < splits; s0 += 4) {
                        float t[G][4];
#pragma unroll
                        for (int u = 0; u < G; ++u)
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                t[u][q] = (j0 + u < M && s0 + q < splits)
                                              ? __ldcg(all + ((long long)(s0 + q) * m_pad + j0 + u) * 128) : 0.f;
#pragma unroll
                        for (int u = 0; u < G; ++u)
#pragma unroll
                            for (int q = 0; q < 4; ++q) v[u] += t[u][q];
                    }
#pragma unroll
                    for (int u = 0; u < G; ++u)
                        if (j0 + u < M) swap_store<EPI>(v[u], old[u], row, j0 + u, N, bias, out, ldo);
                }
                if (threadIdx.x == 64) counters[tile * gridDim.y + blockIdx.y] = 0u;   // ready for the next launch
            }
            }   // counters: this kernel folds
        }
        }   // R == 1
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side: tensor maps ---------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

struct MapKey {
    const void* ptr; int rows, cols, box_rows, box_cols, ld, elem_bytes;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols &&
               ld == o.ld && elem_bytes == o.elem_bytes;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols * 7919u) ^ (size_t)k.box_rows ^
               ((size_t)k.box_cols << 20) ^ ((size_t)k.ld * 31u) ^ ((size_t)k.elem_bytes << 28);
    }
};

// A [rows][cols] row-major matrix (rows `ld` elements apart, bfloat16 or float) seen as boxes of
// box_rows x box_cols elements, swizzled over the box's row bytes (32, 64 or 128).
static bool tensor_map_any(const void* ptr, int rows, int cols, int ld, int elem_bytes, int box_rows, int box_cols,
                           CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey key{ptr, rows, cols, box_rows, box_cols, ld, elem_bytes};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("axon_gemm_tc: cuTensorMapEncodeTiled is not available from this driver"); return false; }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    const int row_bytes = box_cols * elem_bytes;
    const CUtensorMapSwizzle swz = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    CUtensorMap m;
    CUresult r = fn(&m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                    const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("axon_gemm_tc: cuTensorMapEncodeTiled failed with %d (rows %d cols %d)", (int)r, rows, cols); return false; }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}
// An operand: [rows][cols] contiguous bfloat16 in boxes of box_rows x 64.
static bool tensor_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
    return tensor_map_any(ptr, rows, cols, cols, 2, box_rows, TC_BK, out);
}

template <int BN, int STAGES, int RM, bool TMA_OUT>
static int launch_tc(int epi, const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mo, const float* bias,
                     void* out, int M, int N, int K, int ldo, uint32_t stuck_wait_limit, cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * (RM * TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024;
    static_assert(smem >= 8 * 8192 + 1024, "the epilogue stages its chunks in the ring");
    const int m_tiles = (M + RM * TC_BM - 1) / (RM * TC_BM), n_tiles = (N + BN - 1) / BN;
    const dim3 grid((unsigned)(m_tiles * n_tiles)), block(TC_THREADS);
#define AXON_TC_LAUNCH(E)                                                                                          \
    {                                                                                                              \
        if (int st = ensure_dynamic_smem<gemm_tc_kernel<BN, STAGES, E, RM, TMA_OUT>>(smem, "axon_gemm_tc")) return st; \
        launch_pdl(gemm_tc_kernel<BN, STAGES, E, RM, TMA_OUT>, grid, block, smem, stream, ma, mw, mo, bias, out, M, N, K, ldo, m_tiles, stuck_wait_limit); \
    }
    switch (epi) {
        case TC_STORE_F32: AXON_TC_LAUNCH(TC_STORE_F32) break;
        case TC_STORE_BF16: AXON_TC_LAUNCH(TC_STORE_BF16) break;
        case TC_RESIDUAL: AXON_TC_LAUNCH(TC_RESIDUAL) break;
        case TC_SWIGLU: AXON_TC_LAUNCH(TC_SWIGLU) break;
        default: set_error("axon_gemm_tc: unknown epilogue %d", epi); return AXON_BAD_ARGUMENT;
    }
#undef AXON_TC_LAUNCH
    return launch_status("axon_gemm_tc");
}

// The tile shape for a product: among (rows 128 or 256) x (columns 128, 192, 224, 256) the one
// with the least modelled time.  What bounds this kernel is the feed of operands from L2: an SM
// pulls at most about 99 GB/s, and all SMs together about 12.9 TB/s (87 GB/s each when every SM
// has a tile); a tile needs (rows + columns) * K * 2 bytes.  So a wave of tiles takes the bytes
// of one tile over the rate an SM gets with that many SMs busy (or the tile's math at 15.2
// TFLOP/s an SM, which never binds for these shapes), and a launch takes its full waves, its
// last partial wave, and 3 us a wave.  Measured against every shape at the 7B, 1.5B and 32B
// widths with 2,048 and 8,192 rows: the model is within 5 % of the times, and its choice within
// 7 % of the best shape (before, with a model fitted at the 7B widths only, up to 15 % off at
// K = 8,960 and K = 27,648).  It picks 256 x 224 where that fills 128 SMs instead of 112 (3584
// columns: 186 us against 197 us at K = 18944) and 256 x 256 for 4608 and 37888 columns.
struct TileShape { int rm, bn; };
static double modelled_time(int M, int N, int K, int rows, int bn) {
    const long long tiles = (long long)((M + rows - 1) / rows) * ((N + bn - 1) / bn);
    const double bytes = (double)(rows + bn) * K * 2, math = (double)rows * bn * K * 2 / 15.2e12;
    const long long full = tiles / 148, rest = tiles % 148;
    auto wave = [&](long long busy) {
        const double rate = 12.9e12 / (double)busy < 99e9 ? 12.9e12 / (double)busy : 99e9;
        const double feed = bytes / rate;
        return (feed > math ? feed : math) + 3e-6;
    };
    return (double)full * wave(148) + (rest ? wave(rest) : 0.0);
}
static TileShape choose_tile(int M, int N, int K) {
    const int bns[4] = {256, 224, 192, 128};
    TileShape best{1, 256};
    double best_t = 1e30;
    for (int rm = (M > TC_BM ? 2 : 1); rm >= 1; --rm) {
        for (int bn : bns) {
            const double t = modelled_time(M, N, K, rm * TC_BM, bn);
            if (t < best_t * 0.98) { best_t = t; best = TileShape{rm, bn}; }
        }
    }
    return best;
}


// How the swapped kernel would cut a product: token columns per CTA, blocks of tokens, K slabs.
struct SwapPlan { int ntok, blocks, tiles, splits; bool wide; };
static SwapPlan plan_swapped(int M, int N, int K, int target_ctas, long long partial_floats, int n_counters) {
    SwapPlan p;
    // tokens are the MMA's columns: padded to 16 .. 256, and in blocks of 256 beyond that
    p.ntok = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    p.blocks = (M + p.ntok - 1) / p.ntok;
    const int m_pad = p.blocks * p.ntok, tiles128 = (N + 127) / 128, k_total = (K + TC_BK - 1) / TC_BK;
    // many rows: 256-row tiles halve the CTA count (no split then)
    // (measured at 7B sizes: with 2 x target tiles, two 128-row CTAs per SM and six stages beat
    // one 256-row CTA with three; the wide tile pays off only from several waves on)
    p.wide = p.ntok <= 32 && target_ctas > 0 && tiles128 >= 4 * target_ctas;
    p.tiles = p.wide ? (N + 255) / 256 : tiles128;
    // few rows: as many K slabs as it takes to have about `target_ctas` CTAs, each at least 4 stages long
    p.splits = 1;
    if (!p.wide && partial_floats > 0 && p.tiles * p.blocks <= n_counters && p.tiles * p.blocks < target_ctas) {
        p.splits = (target_ctas + p.tiles * p.blocks / 2) / (p.tiles * p.blocks);
        if (p.splits > k_total / 4) p.splits = k_total / 4;
        const long long fit = partial_floats / ((long long)p.tiles * m_pad * 128);
        if (p.splits > fit) p.splits = (int)fit;
        if (p.splits < 1) p.splits = 1;
    }
    const int per_split = (k_total + p.splits - 1) / p.splits;
    p.splits = (k_total + per_split - 1) / per_split;
    return p;
}

// Modelled time of the swapped kernel inside a chain of kernels: a fixed 5.5 us, the weights at
// the rate of memory (a block of 256 tokens beyond the first re-reads them from L2 at about a
// third of that cost), and per token row what the epilogue moves: N * splits * 8 bytes at about
// 1 TB/s (partial sums written and read back; unsplit, the scattered stores of the transposed
// tile cost about as much).  A split product that leaves its partial sums to the reader of its
// output (`deferred`) only writes them, all CTAs at once: N * splits * 4 bytes at about 3.3 TB/s
// (the reader's share is in the fixed part).  Many rows are bound by the MMAs instead, at about
// 0.7 PFLOP/s (0.9 deferred).  Fitted to captured chains of each product of the 1.5B, 7B and 32B widths at
// 32 .. 1,024 rows, and to decode steps of 64 .. 256 requests for the deferred products.
static double modelled_time_swapped(int M, int N, int K, int target_ctas, bool deferred) {
    const SwapPlan p = plan_swapped(M, N, K, target_ctas, 1LL << 40, 1 << 30);
    const double weights = (double)N * K * 2 / 6.5e12 * (1.0 + 0.3 * (p.blocks - 1));
    const double rows = (double)M * N * p.splits * ((deferred && p.splits > 1) ? 1.2e-12 : 8e-12);
    // (the transposed epilogue that folds or applies SwiGLU itself costs the MMAs' rate a fifth more)
    const double math = 2.0 * M * N * K / ((deferred && p.splits > 1) ? 0.9e15 : 0.7e15);
    const double mem = weights + rows;
    return 5.5e-6 + (mem > math ? mem : math);
}
static double modelled_time_tiled(int M, int N, int K) {
    const TileShape ts = choose_tile(M, N, K);
    // never faster than reading the operands once from memory (few rows of a wide product)
    const double tiles = modelled_time(M, N, K, ts.rm * TC_BM, ts.bn), once = ((double)N + M) * K * 2 / 6.5e12 + 3e-6;
    return tiles > once ? tiles : once;
}

}  // namespace axon

using namespace axon;

// Which of the two kernels a product should take: nonzero for the swapped one (axon_gemm_tc_small).
// Up to 32 rows always (decode steps: the token columns are narrow and nothing else comes close);
// beyond 1,024 never (it does not take them); between, whichever the two models call faster.
// `deferred`: the caller lets a split product leave its partial sums to the reader of the output.
AXON_API int axon_gemm_prefers_swapped(int M, int N, int K, int target_ctas, int deferred) {
    if (M <= 32) return 1;
    if (M > 1024) return 0;
    return modelled_time_swapped(M, N, K, target_ctas, deferred != 0) < modelled_time_tiled(M, N, K) ? 1 : 0;
}
// The models' times in microseconds (kind 0: swapped, 1: tiled, 2: swapped and deferred), for tests and reports.
AXON_API double axon_gemm_modelled_us(int kind, int M, int N, int K, int target_ctas) {
    return 1e6 * (kind == 1 ? modelled_time_tiled(M, N, K) : modelled_time_swapped(M, N, K, target_ctas, kind == 2));
}

// For tests and measurements: force the tile shape (rows 1 or 2 times 128; columns 128, 192,
// 224 or 256); rm 0 gives the choice back to the model.
static int g_force_rm = 0, g_force_bn = 0, g_force_plain_out = 0;
static uint32_t g_stuck_wait_limit = 0;
AXON_API void axon_gemm_tc_force_tile(int rm, int bn) { g_force_rm = rm; g_force_bn = bn; }
// For tests: nonzero makes every output take the stores from registers, as outputs that TMA
// cannot address do.
AXON_API void axon_gemm_tc_force_plain_out(int on) { g_force_plain_out = on; }

// a [M][K], w [N][K] bfloat16, contiguous, K % 8 == 0, 16-byte aligned.  Epilogues:
// 0 float out, 1 bfloat16 out, 2 out += (float), 3 SwiGLU to bfloat16 [M][N/2].
AXON_API int axon_gemm_tc(const void* a, const void* w, const float* bias, void* out, int epilogue, int M, int N,
                          int K, int ldo, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return AXON_OK;
    if (K <= 0 || K % 8) { set_error("axon_gemm_tc: K %d must be a positive multiple of 8", K); return AXON_BAD_ARGUMENT; }
    if (((uintptr_t)a | (uintptr_t)w) & 15) { set_error("axon_gemm_tc: operands must be 16-byte aligned"); return AXON_BAD_ARGUMENT; }
    if (epilogue == TC_SWIGLU && (N % 2)) { set_error("axon_gemm_tc: SwiGLU needs an even number of columns"); return AXON_BAD_ARGUMENT; }
    TileShape ts = choose_tile(M, N, K);
    if (g_force_rm > 0) ts = TileShape{g_force_rm, g_force_bn};
    CUtensorMap ma, mw, mo;
    if (!tensor_map(a, M, K, ts.rm * TC_BM, &ma) || !tensor_map(w, N, K, ts.bn, &mw)) return AXON_BAD_ARGUMENT;
    // the output through TMA when it can address it: 16-byte aligned base and rows (else from registers)
    const int out_bytes = (epilogue == TC_STORE_BF16 || epilogue == TC_SWIGLU) ? 2 : 4;
    const int out_cols = epilogue == TC_SWIGLU ? N / 2 : N;
    const bool tma_out = !g_force_plain_out && ((uintptr_t)out & 15) == 0 && ((long long)ldo * out_bytes) % 16 == 0;
    if (tma_out) {
        if (!tensor_map_any(out, M, out_cols, ldo, out_bytes, 32, epilogue == TC_SWIGLU ? 16 : 32, &mo)) return AXON_BAD_ARGUMENT;
    } else {
        mo = ma;
    }
#define AXON_TC_ARGS epilogue, ma, mw, mo, bias, out, M, N, K, ldo, g_stuck_wait_limit, stream
#define AXON_TC_SHAPE(BN, STAGES, RM) return tma_out ? launch_tc<BN, STAGES, RM, true>(AXON_TC_ARGS) : launch_tc<BN, STAGES, RM, false>(AXON_TC_ARGS)
    if (ts.rm == 2) {
        switch (ts.bn) {
            case 256: AXON_TC_SHAPE(256, 3, 2);
            case 224: AXON_TC_SHAPE(224, 3, 2);
            case 192: AXON_TC_SHAPE(192, 4, 2);
            default: AXON_TC_SHAPE(128, 4, 2);
        }
    }
    switch (ts.bn) {
        case 256: AXON_TC_SHAPE(256, 4, 1);
        case 224: AXON_TC_SHAPE(224, 4, 1);
        case 192: AXON_TC_SHAPE(192, 5, 1);
        default: AXON_TC_SHAPE(128, 6, 1);
    }
#undef AXON_TC_SHAPE
#undef AXON_TC_ARGS
}

namespace axon {
template <int NTOK, int STAGES, int R>
static int launch_swap(int epi, const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* out,
                       float* partial, unsigned int* counters, int M, int N, int K, int ldo, int tiles, int splits,
                       int per_split, cudaStream_t stream) {
    constexpr size_t smem = (size_t)STAGES * (R * 128 * TC_BK * 2 + NTOK * TC_BK * 2) + 1024;
    static_assert(smem <= 227 * 1024, "the ring does not fit shared memory");
    const dim3 grid((unsigned)(tiles * splits), (unsigned)((M + NTOK - 1) / NTOK)), block(192);
#define AXON_SWAP_LAUNCH(E)                                                                                        \
    {                                                                                                              \
        if (int st = ensure_dynamic_smem<gemm_tc_swap_kernel<NTOK, STAGES, E, R>>(smem, "axon_gemm_tc_small")) return st; \
        launch_pdl(gemm_tc_swap_kernel<NTOK, STAGES, E, R>, grid, block, smem, stream, mw, mx, bias, out, partial, counters, M, N, K, ldo, splits, per_split); \
    }
    switch (epi) {
        case TC_STORE_F32: AXON_SWAP_LAUNCH(TC_STORE_F32) break;
        case TC_STORE_BF16: AXON_SWAP_LAUNCH(TC_STORE_BF16) break;
        case TC_RESIDUAL: AXON_SWAP_LAUNCH(TC_RESIDUAL) break;
        case TC_SWIGLU: AXON_SWAP_LAUNCH(TC_SWIGLU) break;
        default: set_error("axon_gemm_tc_small: unknown epilogue %d", epi); return AXON_BAD_ARGUMENT;
    }
#undef AXON_SWAP_LAUNCH
    return launch_status("axon_gemm_tc_small");
}
}  // namespace axon

// The product for at most 1024 activation rows (see gemm_tc_swap_kernel): the weights are read
// once per block of 256 tokens, which beats the 256 x 256 tiles of axon_gemm_tc while the
// product is bound by reading weights and its tiles would not fill the machine.  `partial` is
// scratch for split-K partial tiles (`partial_floats` floats; 0 forbids splitting) and
// `counters` an array of `n_counters` zeroed 32-bit counters that the kernel leaves zeroed.
// `target_ctas` is the number of CTAs to aim at (the SM count works best: one CTA per SM
// leaves room for the next kernel's CTAs to preload their weights).  Operands as in
// axon_gemm_tc.  Calls that share the scratch must not overlap on the GPU.
// `defer` (store-float and residual epilogues): when the product is split, leave the partial
// sums in `partial` for the reader of the output (SplitFold: axon_rmsnorm_fold,
// axon_rope_kv_write, axon_fold_partials), which must run before `partial` is written again;
// bias and residual are then the reader's to add and `out` is not touched.
// `plan` (may be null) receives {splits, token rows of the partial tiles (M padded), deferred 0/1}.
AXON_API int axon_gemm_tc_small(const void* a, const void* w, const float* bias, void* out, int epilogue, int M,
                                int N, int K, int ldo, float* partial, long long partial_floats,
                                unsigned int* counters, int n_counters, int target_ctas, int defer, int* plan,
                                cudaStream_t stream) {
    if (M <= 0 || N <= 0) return AXON_OK;
    if (M > 1024) { set_error("axon_gemm_tc_small: %d rows; this kernel takes at most 1024", M); return AXON_BAD_ARGUMENT; }
    if (K <= 0 || K % 8) { set_error("axon_gemm_tc_small: K %d must be a positive multiple of 8", K); return AXON_BAD_ARGUMENT; }
    if (((uintptr_t)a | (uintptr_t)w) & 15) { set_error("axon_gemm_tc_small: operands must be 16-byte aligned"); return AXON_BAD_ARGUMENT; }
    if (epilogue == TC_SWIGLU && (N % 2)) { set_error("axon_gemm_tc_small: SwiGLU needs an even number of columns"); return AXON_BAD_ARGUMENT; }
    const SwapPlan sp = plan_swapped(M, N, K, target_ctas, (partial != nullptr && counters != nullptr) ? partial_floats : 0, n_counters);
    const int ntok = sp.ntok, m_pad = sp.blocks * sp.ntok, tiles = sp.tiles, splits = sp.splits;
    const bool wide = sp.wide;
    const int k_total = (K + TC_BK - 1) / TC_BK, per_split = (k_total + splits - 1) / splits;
    const bool deferred = defer && splits > 1 && (epilogue == TC_STORE_F32 || epilogue == TC_RESIDUAL);
    if (plan) { plan[0] = splits; plan[1] = m_pad; plan[2] = deferred ? 1 : 0; }
    if (deferred) counters = nullptr;                 // the kernel stops after writing its partial tile
    CUtensorMap mw, mx;
    if (!tensor_map(w, N, K, wide ? 256 : 128, &mw) || !tensor_map(a, M, K, ntok, &mx)) return AXON_BAD_ARGUMENT;
#define AXON_SWAP_ARGS epilogue, mw, mx, bias, out, partial, counters, M, N, K, ldo, tiles, splits, per_split, stream
    if (ntok == 16) return wide ? launch_swap<16, 3, 2>(AXON_SWAP_ARGS) : launch_swap<16, 6, 1>(AXON_SWAP_ARGS);
    if (ntok == 32) return wide ? launch_swap<32, 3, 2>(AXON_SWAP_ARGS) : launch_swap<32, 5, 1>(AXON_SWAP_ARGS);
    if (ntok == 64) return launch_swap<64, 4, 1>(AXON_SWAP_ARGS);
    if (ntok == 128) return launch_swap<128, 5, 1>(AXON_SWAP_ARGS);
    return launch_swap<256, 4, 1>(AXON_SWAP_ARGS);
#undef AXON_SWAP_ARGS
}

// For the test of the failure path: while `polls` != 0, axon_gemm_tc launches its kernel so that the
// epilogue's wait for the accumulator is never answered and gives up after that many polls (the
// output is then garbage and the status word reads 3).  0 restores normal launches.
AXON_API void axon_gemm_tc_test_stuck_wait(unsigned int polls) { g_stuck_wait_limit = polls; }

// Clears the status word (after a test of the failure path, or once a failure has been reported).
AXON_API int axon_gemm_tc_clear_status() {
    const unsigned int zero = 0;
    return cudaMemcpyToSymbol(g_tc_error, &zero, sizeof zero) == cudaSuccess ? AXON_OK : AXON_CUDA_ERROR;
}

// 0 when no kernel of this file ever gave up on a wait; else 1 + the role (0 producer,
// 1 MMA, 2 epilogue).  Synchronises the device.
AXON_API int axon_gemm_tc_status() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof v) != cudaSuccess) return -1;
    return (int)v;
}
