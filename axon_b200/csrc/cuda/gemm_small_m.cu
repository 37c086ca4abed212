// Products with few activation rows (decode steps): out[m][n] = sum_k a[m][k] w[n][k].
//
// With 1..64 tokens a product is bound by reading the weights once from HBM.  A CTA
// owns 16 weight rows; its 8 warps split K into interleaved 64-wide chunks and stream
// their chunks with 16-byte loads (three stages in flight per thread), multiply on the
// tensor cores with the weights as the 16-row operand of mma.m16n8k16 and up to 64
// tokens as 8-wide column tiles, and reduce across warps through shared memory in a
// fixed order.  The k index is permuted inside a 64-wide chunk so that every thread
// loads whole 16-byte pieces of a row (the contraction does not care about the order
// as long as both operands agree).
//
// Epilogues: store (float or bfloat16) with optional bias; add into a float residual;
// SwiGLU on interleaved gate/up rows (row 2j gate, 2j+1 up) to bfloat16.
//
// Needs K % 8 == 0 (16-byte row pieces) and M <= 64; anything else is refused and the
// caller takes the plain kernel.
#include "common.cuh"

namespace axon {

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

enum { EPI_STORE_F32 = 0, EPI_STORE_BF16 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3 };

constexpr int SM_ROWS = 16, SM_WARPS = 8, SM_KCHUNK = 64, SM_STAGES = 3;

struct WeightRegs {
    uint4 lo[2];  // row g:     elements k0 + 8t .. + 7 and k0 + 32 + 8t .. + 7
    uint4 hi[2];  // row g + 8
};

template <int NT, int EPI>
__global__ void __launch_bounds__(SM_WARPS * 32)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w,
                    const float* __restrict__ bias, void* __restrict__ out, int M, int N, int K, int lda,
                    int ldo) {
    __shared__ float red[SM_WARPS][SM_ROWS][NT * 8 + 1];
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * SM_ROWS;
    const int r_lo = min(row0 + g, N - 1), r_hi = min(row0 + g + 8, N - 1);
    const __nv_bfloat16* w_lo = w + (long long)r_lo * K + 8 * t;
    const __nv_bfloat16* w_hi = w + (long long)r_hi * K + 8 * t;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

    auto load_w = [&](WeightRegs& r, int k0) {
        // the thread's two 8-element pieces start at k0 + 8t and k0 + 32 + 8t, so the four
        // threads of a row read two whole 64-byte runs; pieces past K read as zero
        const int ka = k0 + 8 * t;
        r.lo[0] = (ka + 8 <= K) ? ldg_stream(w_lo + k0) : zero4;
        r.lo[1] = (ka + 40 <= K) ? ldg_stream(w_lo + k0 + 32) : zero4;
        r.hi[0] = (ka + 8 <= K) ? ldg_stream(w_hi + k0) : zero4;
        r.hi[1] = (ka + 40 <= K) ? ldg_stream(w_hi + k0 + 32) : zero4;
    };

    const int kstep = SM_WARPS * SM_KCHUNK;
    WeightRegs st[SM_STAGES];
    int k_load = warp * SM_KCHUNK;
#pragma unroll
    for (int s = 0; s < SM_STAGES; ++s) {
        if (k_load < K) load_w(st[s], k_load);
        k_load += kstep;
    }
    // the weights above do not depend on the kernel before this one; the activations do
    pdl_wait();
    for (int k0 = warp * SM_KCHUNK; k0 < K; k0 += SM_STAGES * kstep) {
#pragma unroll
        for (int s = 0; s < SM_STAGES; ++s) {
            const int kc = k0 + s * kstep;
            if (kc < K) {
                const WeightRegs cur = st[s];
                if (k_load < K) load_w(st[s], k_load);
                k_load += kstep;
                const int ka = kc + 8 * t;
                const uint32_t wl[8] = {cur.lo[0].x, cur.lo[0].y, cur.lo[0].z, cur.lo[0].w,
                                        cur.lo[1].x, cur.lo[1].y, cur.lo[1].z, cur.lo[1].w};
                const uint32_t wh[8] = {cur.hi[0].x, cur.hi[0].y, cur.hi[0].z, cur.hi[0].w,
                                        cur.hi[1].x, cur.hi[1].y, cur.hi[1].z, cur.hi[1].w};
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int tok = j * 8 + g;
                    uint4 x0 = zero4, x1 = zero4;
                    if (tok < M) {
                        const __nv_bfloat16* ap = a + (long long)tok * lda + ka;
                        if (ka + 8 <= K) x0 = ldg_cached(ap);
                        if (ka + 40 <= K) x1 = ldg_cached(ap + 32);
                    }
                    const uint32_t xb[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        mma_bf16(acc[j], wl[2 * i], wh[2 * i], wl[2 * i + 1], wh[2 * i + 1], xb[2 * i], xb[2 * i + 1]);
                }
            }
        }
    }

    // partial sums of the 8 warps -> shared memory, then summed in warp order
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        red[warp][g][j * 8 + 2 * t] = acc[j][0];
        red[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
        red[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
        red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    if (EPI == EPI_SWIGLU) {
        // 8 output columns (pairs of rows) x tokens
        for (int e = threadIdx.x; e < (SM_ROWS / 2) * NT * 8; e += blockDim.x) {
            const int pr = e % (SM_ROWS / 2), tok = e / (SM_ROWS / 2);
            const int row = row0 + 2 * pr;
            if (tok >= M || row + 1 >= N) continue;
            float gv = 0.f, uv = 0.f;
#pragma unroll
            for (int wi = 0; wi < SM_WARPS; ++wi) {
                gv += red[wi][2 * pr][tok];
                uv += red[wi][2 * pr + 1][tok];
            }
            if (bias) { gv += bias[row]; uv += bias[row + 1]; }
            const float v = gv / (1.0f + expf(-gv)) * uv;
            ((__nv_bfloat16*)out)[(long long)tok * ldo + (row >> 1)] = __float2bfloat16_rn(v);
        }
    } else {
        for (int e = threadIdx.x; e < SM_ROWS * NT * 8; e += blockDim.x) {
            const int r = e % SM_ROWS, tok = e / SM_ROWS;
            const int row = row0 + r;
            if (tok >= M || row >= N) continue;
            float v = 0.f;
#pragma unroll
            for (int wi = 0; wi < SM_WARPS; ++wi) v += red[wi][r][tok];
            if (bias) v += bias[row];
            const long long o = (long long)tok * ldo + row;
            if (EPI == EPI_STORE_F32) ((float*)out)[o] = v;
            else if (EPI == EPI_STORE_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v);
            else ((float*)out)[o] += v;
        }
    }
}

template <int NT>
static int launch_small_m(int epi, const void* a, const void* w, const float* bias, void* out, int M, int N,
                          int K, int lda, int ldo, cudaStream_t stream) {
    const dim3 grid((N + SM_ROWS - 1) / SM_ROWS), block(SM_WARPS * 32);
    const __nv_bfloat16* ap = (const __nv_bfloat16*)a;
    const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
    switch (epi) {
        case EPI_STORE_F32: launch_pdl(gemm_small_m_kernel<NT, EPI_STORE_F32>, grid, block, 0, stream, ap, wp, bias, out, M, N, K, lda, ldo); break;
        case EPI_STORE_BF16: launch_pdl(gemm_small_m_kernel<NT, EPI_STORE_BF16>, grid, block, 0, stream, ap, wp, bias, out, M, N, K, lda, ldo); break;
        case EPI_RESIDUAL: launch_pdl(gemm_small_m_kernel<NT, EPI_RESIDUAL>, grid, block, 0, stream, ap, wp, bias, out, M, N, K, lda, ldo); break;
        case EPI_SWIGLU: launch_pdl(gemm_small_m_kernel<NT, EPI_SWIGLU>, grid, block, 0, stream, ap, wp, bias, out, M, N, K, lda, ldo); break;
        default: set_error("axon_gemm_small_m: unknown epilogue %d", epi); return AXON_BAD_ARGUMENT;
    }
    return launch_status("axon_gemm_small_m");
}

}  // namespace axon

using namespace axon;

// a [M][K] bfloat16 (row stride lda), w [N][K] bfloat16, M <= 64, K % 8 == 0.
// epilogue: 0 float out, 1 bfloat16 out, 2 out += (float), 3 SwiGLU of interleaved rows
// to bfloat16 [M][N/2].  ldo is the row stride of out in elements.
AXON_API int axon_gemm_small_m(const void* a, const void* w, const float* bias, void* out, int epilogue,
                               int M, int N, int K, int lda, int ldo, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return AXON_OK;
    if (M > 64) { set_error("axon_gemm_small_m: %d rows; this kernel takes at most 64", M); return AXON_BAD_ARGUMENT; }
    if (K <= 0 || K % 8 || lda % 8) { set_error("axon_gemm_small_m: K %d and the row stride %d must be multiples of 8", K, lda); return AXON_BAD_ARGUMENT; }
    if (((uintptr_t)a | (uintptr_t)w) & 15) { set_error("axon_gemm_small_m: operands must be 16-byte aligned"); return AXON_BAD_ARGUMENT; }
    if (epilogue == EPI_SWIGLU && (N % 2)) { set_error("axon_gemm_small_m: SwiGLU needs an even number of rows"); return AXON_BAD_ARGUMENT; }
    if (M <= 8) return launch_small_m<1>(epilogue, a, w, bias, out, M, N, K, lda, ldo, stream);
    if (M <= 16) return launch_small_m<2>(epilogue, a, w, bias, out, M, N, K, lda, ldo, stream);
    if (M <= 32) return launch_small_m<4>(epilogue, a, w, bias, out, M, N, K, lda, ldo, stream);
    return launch_small_m<8>(epilogue, a, w, bias, out, M, N, K, lda, ldo, stream);
}
