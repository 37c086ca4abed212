// A measuring kernel, not part of any model: how many cycles the tensor pipe of an SM spends on
// the products of the prompt attention kernel as that kernel issues them (same shapes, operand
// layouts and shared-memory footprints; every operand element is 1.0 or 0.5, since operands of
// zeros or of arbitrary bit patterns gave other times).
// One thread issues the score products of a 64-key step (two sub-tiles of 128 query rows: 16
// tcgen05.mma of M 128, N 64, K 16), another the value products (8 of M 128, N 128, K 16), each
// into its own tensor-memory columns and without waiting for anything, so what is timed is the
// pipe and its operand fetch alone.  Every wait is bounded and tensor memory is freed on every path.
#include "tcgen05.cuh"

namespace axon {

// what: bit 0 score products; bit 1 value products with P in shared memory and V MN-major (as V
// lies in the cache); bit 2 the same with P in tensor memory; bit 3 products of the value
// products' shape (M 128, N 128, K 16, 8 a step) with both operands K-major from shared memory
// (the queries against 128 keys), to tell the operand layout's share of their time.
__global__ void __launch_bounds__(128, 1) mma_probe_kernel(int steps, int what, unsigned long long* cycles) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = ((uint32_t)__cvta_generic_to_shared(smem_dyn) + 1023u) & ~1023u;
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&bars[0]);
    for (uint32_t i = threadIdx.x; i < 192 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(smem_dyn)[i] = 0x3F803F80u;   // 1.0, 1.0
    if (threadIdx.x == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"((uint32_t)__cvta_generic_to_shared(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    {
        // tensor memory starts defined: P (columns 0..255) 0.5 everywhere, the accumulators zero
        uint32_t half[32], zero[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) { half[i] = 0x3F003F00u; zero[i] = 0u; }
        const uint32_t lanes = tmem + ((uint32_t)(warp * 32) << 16);
        for (int c = 0; c < 8; ++c) tmem_st32(lanes + (uint32_t)(c * 32), half);
        for (int c = 8; c < 16; ++c) tmem_st32(lanes + (uint32_t)(c * 32), zero);
        tmem_st_wait();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }
    // Q: two sub-tiles of 32 KB; keys: three stages of 16 KB (two adjacent ones serve the 128-key form);
    // values: three stages; P: two tiles of 16 KB
    const uint32_t q_sm = base, k_sm = base + 65536, v_sm = k_sm + 3 * 16384, p_sm = v_sm + 3 * 16384;
    const long long t0 = clock64();
    if (lane == 0 && warp == 2 && (what & 8)) {
        for (int t = 0; t < steps; ++t) {
            for (int g = 0; g < 2; ++g) {
                const uint32_t qg = q_sm + (uint32_t)g * 32768;
#pragma unroll
                for (int k = 0; k < 4; ++k)           // half a head's dimensions: 4 MMAs, as a value product of 64 keys has
                    umma(tmem + 256 + (uint32_t)(g * 128), smem_desc(qg) + (uint64_t)(2 * k), smem_desc(k_sm) + (uint64_t)(2 * k), instr_desc(128, 128), (t | k) ? 1u : 0u);
            }
        }
        umma_commit(bar0 + 8);
        mbar_wait(bar0 + 8, 0, 1);
        if (blockIdx.x == 0) cycles[1] = (unsigned long long)(clock64() - t0);
    }
    if (lane == 0 && warp == 0 && (what & 1)) {
        // (where the value products read P from tensor memory the scores land over it, as in the
        // kernel, and P is then 128.0 and 0.0 instead of 0.5: ordinary numbers either way)
        for (int t = 0; t < steps; ++t) {
            const uint32_t kt = k_sm + (uint32_t)(t % 3) * 16384;
            for (int g = 0; g < 2; ++g) {
                const uint32_t qg = q_sm + (uint32_t)g * 32768;
                const uint32_t d = tmem + (uint32_t)((2 * g + (t & 1)) * 64);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma(d, smem_desc(qg + (uint32_t)(k >> 2) * (128 * 128)) + (uint64_t)(2 * (k & 3)),
                         smem_desc(kt + (uint32_t)(k >> 2) * (64 * 128)) + (uint64_t)(2 * (k & 3)), instr_desc(128, 64), k ? 1u : 0u);
            }
        }
        umma_commit(bar0);
        mbar_wait(bar0, 0, 1);
        if (blockIdx.x == 0) cycles[0] = (unsigned long long)(clock64() - t0);
    }
    if (lane == 0 && warp == 1 && (what & (2 | 4))) {
        for (int t = 0; t < steps; ++t) {
            const uint32_t vt = v_sm + (uint32_t)(t % 3) * 16384;
            for (int g = 0; g < 2; ++g) {
                const uint32_t d = tmem + 256 + (uint32_t)(g * 128), pg = p_sm + (uint32_t)g * 16384;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t v_mn = smem_desc_mn(vt + (uint32_t)k * 2048u, 64 * 128);
                    if (what & 2) umma(d, smem_desc(pg) + (uint64_t)(2 * k), v_mn, instr_desc_b_mn(128, 128), (t | k) ? 1u : 0u);
                    else umma_ta(d, tmem + (uint32_t)((2 * g + (t & 1)) * 64 + 8 * k), v_mn, instr_desc_b_mn(128, 128), (t | k) ? 1u : 0u);
                }
            }
        }
        umma_commit(bar0 + 8);
        mbar_wait(bar0 + 8, 0, 1);
        if (blockIdx.x == 0) cycles[1] = (unsigned long long)(clock64() - t0);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

}  // namespace axon

using namespace axon;

// Runs the probe on every SM (`what` as above, `steps` 64-key steps) and returns the cycles the
// thread of the score products (cycles[0]) and of the value products (cycles[1]) took on the first
// SM; 0 for a thread that issued nothing.  `scratch`: 16 bytes of device memory.
AXON_API int axon_mma_probe(int what, int steps, unsigned long long* scratch, unsigned long long* cycles, cudaStream_t stream) {
    if (steps < 1 || steps > 100000 || scratch == nullptr || cycles == nullptr) { set_error("axon_mma_probe: bad arguments"); return AXON_BAD_ARGUMENT; }
    constexpr size_t smem = 193 * 1024;
    if (int st = ensure_dynamic_smem<mma_probe_kernel>(smem, "axon_mma_probe")) return st;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaMemsetAsync(scratch, 0, 16, stream);
    mma_probe_kernel<<<sms, 128, smem, stream>>>(steps, what, scratch);
    if (cudaStreamSynchronize(stream) != cudaSuccess) return launch_status("axon_mma_probe");
    if (cudaMemcpy(cycles, scratch, 16, cudaMemcpyDeviceToHost) != cudaSuccess) return launch_status("axon_mma_probe");
    unsigned int flag = 0;
    cudaMemcpyFromSymbol(&flag, g_tc_error, sizeof flag);
    if (flag) { set_error("axon_mma_probe: a wait gave up (role %u)", flag - 1); return AXON_CUDA_ERROR; }
    return launch_status("axon_mma_probe");
}
