// Plain kernels of every op, templated on the element type.
//
// These run the whole model in true 32-bit (float weights, activations and cache,
// FFMA products, no tensor-core mode of any kind) and are the slow-but-general
// fallbacks of the bfloat16 path for sizes its tuned kernels refuse.  Each output
// is reduced in an order that depends only on its own row (ascending k in a
// product, ascending position in attention), never on what else is in the batch.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>

namespace axon {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

// ---------------------------------------------------------------------------
// Embedding: x[t][:] = table[token[t]][:] widened to float.
template <typename T>
__global__ void embed_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ x, int dim, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const long long row = tokens[t];
    for (int d = threadIdx.x; d < dim; d += blockDim.x)
        x[(long long)t * dim + d] = ldf(table + row * dim + d) * scale;
}

// ---------------------------------------------------------------------------
// RMSNorm: h = x * rsqrt(mean(x^2) + eps) * gain, one block per row.
// `rows` (optional) gathers: output row r is the norm of input row rows[r].
// With `fold` the row first takes the partial products that the product before left for it
// (x[row] += sum of the slabs, written back), so that product needs no pass of its own to add them.
template <typename TO>
__global__ void rmsnorm_kernel(float* x, const float* __restrict__ gain,
                               const int32_t* __restrict__ rows, TO* __restrict__ out, int dim,
                               float eps, int unit_offset, SplitFold fold) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const long long r_in = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + r_in * dim;
    float ss = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float v = xr[d];
        if (fold.partial) {
            v += fold.at((int)r_in, d);
            xr[d] = v;                             // read again below by the same thread
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    TO* o = out + (long long)blockIdx.x * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        const float g = unit_offset ? 1.0f + gain[d] : gain[d];
        stf(o + d, xr[d] * inv * g);
    }
}

// The same for rows of whole float4s (dim % 4 == 0, aligned): a thread keeps its VPT float4s
// of the row and of the gain in registers, so the row is read once and every load is in
// flight before the first is used (the row's latency is paid once, not per element).
__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* o, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(o) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}
template <typename TO, int VPT>
__global__ void __launch_bounds__(1024)
rmsnorm_vec_kernel(float* x, const float* __restrict__ gain, const int32_t* __restrict__ rows,
                   TO* __restrict__ out, int dim, float eps, int unit_offset, SplitFold fold) {
    __shared__ float red[32];
    const int n4 = dim >> 2;
    float4 g[VPT], v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {                // the gain does not depend on the kernel before
        const int i = threadIdx.x + k * blockDim.x;
        g[k] = i < n4 ? reinterpret_cast<const float4*>(gain)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_launch_dependents();
    pdl_wait();
    const long long r_in = rows ? rows[blockIdx.x] : blockIdx.x;
    float4* xr = reinterpret_cast<float4*>(x + r_in * dim);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (fold.partial) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < n4) {
                const float4 f = fold.at4((int)r_in, 4 * i);
                v[k].x += f.x; v[k].y += f.y; v[k].z += f.z; v[k].w += f.w;
                xr[i] = v[k];
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss);
        ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    const float off = unit_offset ? 1.0f : 0.0f;
    TO* o = out + (long long)blockIdx.x * dim;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4)
            store4(o + 4 * i, v[k].x * inv * (off + g[k].x), v[k].y * inv * (off + g[k].y),
                   v[k].z * inv * (off + g[k].z), v[k].w * inv * (off + g[k].w));
    }
}

// ---------------------------------------------------------------------------
// out[m][n] = sum_k a[m][k] * w[n][k] (+ bias[n]); mode 0 stores, mode 1 adds
// into a float residual.  64x64 tile, 16-deep stages, 4x4 outputs per thread;
// every output accumulates k in ascending order.
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA* __restrict__ a, const TW* __restrict__ w, const float* __restrict__ bias,
                  TO* __restrict__ out, int M, int N, int K, int lda, int ldo, int mode) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float sa[BK][BM + 4];
    __shared__ float sw[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 values per operand, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            sa[kk][r] = (gm < M && gk < K) ? ldf(a + (long long)gm * lda + gk) : 0.f;
            sw[kk][r] = (gn < N && gk < K) ? ldf(w + (long long)gn * K + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = sw[kk][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + tm + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tn + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[gn];
            TO* o = out + (long long)gm * ldo + gn;
            if (mode == 1) v += ldf(o);
            stf(o, v);
        }
    }
}

// ---------------------------------------------------------------------------
// SwiGLU on interleaved rows: act[t][j] = silu(gu[t][2j]) * gu[t][2j+1].
template <typename TO>
__global__ void swiglu_kernel(const float* __restrict__ gu, TO* __restrict__ act, long long total,
                              int ffn) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / ffn, j = i % ffn;
    const float g = gu[t * 2 * ffn + 2 * j], u = gu[t * 2 * ffn + 2 * j + 1];
    stf(act + i, g / (1.0f + expf(-g)) * u);
}

// ---------------------------------------------------------------------------
// Rotation table: (cos, sin) of pos * inv_freq[i]; the angle and its sine and
// cosine are taken in double and rounded to float once.
__global__ void rope_table_kernel(const int32_t* __restrict__ positions,
                                  const double* __restrict__ inv_freq, float2* __restrict__ table,
                                  int n, int half, float magnitude) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * half) return;
    const int t = i / half, f = i % half;
    const double ang = (double)positions[t] * inv_freq[f];
    double s, c;
    sincos(ang, &s, &c);
    table[i] = make_float2((float)c * magnitude, (float)s * magnitude);
}

// ---------------------------------------------------------------------------
// Rotate q and k, write q out and k, v into their pages.
// qkv: float [n][q_dim + 2 kv_dim] with biases already added.  The first `rot`
// elements of each head rotate (pairs (i, i + rot/2) when `adjacent` is 0, pairs
// (2i, 2i + 1) otherwise); the rest pass through.
template <typename T>
__global__ void rope_kv_write_kernel(const float* __restrict__ qkv, const float2* __restrict__ table,
                                     const int32_t* __restrict__ positions,
                                     const int32_t* __restrict__ token_slot, T* __restrict__ q_out,
                                     T* __restrict__ pool, PagedKv kv, int heads, int rot, int adjacent,
                                     int write_kv, SplitFold fold) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int hd = kv.head_dim, half = hd / 2, rhalf = rot / 2;
    // a row of the product: q heads and k heads of `hd`, then (two planes) v heads of `v_dim`
    const int q_dim = heads * hd, k_dim = kv.kv_heads * hd;
    const int vhalf = kv.planes == 2 ? kv.v_dim / 2 : 0;
    const int width = q_dim + k_dim + kv.kv_heads * 2 * vhalf;
    const float* row = qkv + (long long)t * width;
    const int pos = positions[t], slot = token_slot[t];
    const int qk_items = (heads + kv.kv_heads) * half;
    const int items = qk_items + kv.kv_heads * vhalf;
    for (int it = blockIdx.y * blockDim.x + threadIdx.x; it < items; it += gridDim.y * blockDim.x) {
        if (it >= qk_items) {
            // a pair of a value row: passed through as it is
            if (!write_kv) continue;
            const int kh = (it - qk_items) / vhalf, i = (it - qk_items) % vhalf;
            const int col = q_dim + k_dim + kh * kv.v_dim + 2 * i;
            const float a = fold.partial ? fold.at(t, col) : row[col];
            const float b = fold.partial ? fold.at(t, col + 1) : row[col + 1];
            T* dst = pool + kv.v_row(slot, pos, kh) + 2 * i;
            stf(dst, a);
            stf(dst + 1, b);
            continue;
        }
        const int h = it / half, i = it % half;
        // element indices of the pair this thread owns
        int ia, ib;
        bool rotate;
        if (table != nullptr && i < rhalf) {
            rotate = true;
            if (adjacent) { ia = 2 * i; ib = 2 * i + 1; } else { ia = i; ib = i + rhalf; }
        } else {
            // beyond the rotated part (or no rotation): pass two elements through
            rotate = false;
            const int j = (table != nullptr) ? (i - rhalf) : i;
            const int base = (table != nullptr) ? rot : 0;
            ia = base + 2 * j; ib = base + 2 * j + 1;
        }
        if (h >= heads && !write_kv) continue;
        const float a = fold.partial ? fold.at(t, h * hd + ia) : row[h * hd + ia];
        const float b = fold.partial ? fold.at(t, h * hd + ib) : row[h * hd + ib];
        float ra = a, rb = b;
        if (rotate) {
            const float2 cs = table[(long long)t * rhalf + i];
            ra = a * cs.x - b * cs.y;
            rb = a * cs.y + b * cs.x;
        }
        T* dst = h < heads ? q_out + (long long)t * q_dim + h * hd : pool + kv.row(slot, pos, h - heads);
        stf(dst + ia, ra);
        stf(dst + ib, rb);
    }
}

// The same for the common layout (pairs (i, i + head/2), the whole head rotated, head % 8 == 0,
// 16-byte aligned rows): a thread owns four consecutive pairs, reads them as float4 and stores
// 8 bytes each, instead of single elements.
template <typename T>
__global__ void rope_kv_write_vec_kernel(const float* __restrict__ qkv, const float2* __restrict__ table,
                                         const int32_t* __restrict__ positions,
                                         const int32_t* __restrict__ token_slot, T* __restrict__ q_out,
                                         T* __restrict__ pool, PagedKv kv, int heads, int write_kv, SplitFold fold) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int hd = kv.head_dim, half = hd / 2, quads = half / 4;
    const int q_dim = heads * hd, kv_dim = kv.kv_heads * hd;
    const float* row = qkv + (long long)t * (q_dim + 2 * kv_dim);
    const int pos = positions[t], slot = token_slot[t];
    const int items = (heads + 2 * kv.kv_heads) * quads;
    for (int it = blockIdx.y * blockDim.x + threadIdx.x; it < items; it += gridDim.y * blockDim.x) {
        const int h = it / quads, i0 = (it % quads) * 4;
        const bool is_q = h < heads, is_v = h >= heads + kv.kv_heads;
        if (!is_q && !write_kv) continue;
        const int col = h * hd;                           // q heads, then k heads, then v heads
        float4 a, b;
        if (fold.partial) { a = fold.at4(t, col + i0); b = fold.at4(t, col + half + i0); }
        else { a = *reinterpret_cast<const float4*>(row + col + i0); b = *reinterpret_cast<const float4*>(row + col + half + i0); }
        float4 ra = a, rb = b;
        if (!is_v) {
            const float4 c01 = *reinterpret_cast<const float4*>(table + (long long)t * half + i0);       // cos0 sin0 cos1 sin1
            const float4 c23 = *reinterpret_cast<const float4*>(table + (long long)t * half + i0 + 2);
            ra.x = a.x * c01.x - b.x * c01.y; rb.x = a.x * c01.y + b.x * c01.x;
            ra.y = a.y * c01.z - b.y * c01.w; rb.y = a.y * c01.w + b.y * c01.z;
            ra.z = a.z * c23.x - b.z * c23.y; rb.z = a.z * c23.y + b.z * c23.x;
            ra.w = a.w * c23.z - b.w * c23.w; rb.w = a.w * c23.w + b.w * c23.z;
        }
        T* dst;
        if (is_q) dst = q_out + (long long)t * q_dim + col;
        else dst = pool + kv.row(slot, pos, is_v ? h - heads - kv.kv_heads : h - heads) + (is_v ? kv.v_offset : 0);
        store4(dst + i0, ra.x, ra.y, ra.z, ra.w);
        store4(dst + half + i0, rb.x, rb.y, rb.z, rb.w);
    }
}

// ---------------------------------------------------------------------------
// Causal attention over the paged cache, one warp per (token, query head).
// Keys kv_begin..pos are folded 32 at a time in ascending order with a running
// maximum; kv_begin = max(0, pos - window + 1) when window > 0.
template <typename T>
__global__ void __launch_bounds__(128)
attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ pool,
                       const int32_t* __restrict__ positions, const int32_t* __restrict__ token_slot,
                       T* __restrict__ out, PagedKv kv, int n_tokens, int heads, float scale,
                       int window) {
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hd = kv.head_dim, vd = kv.v_dim;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    const int group = heads / kv.kv_heads, kh = h / group;
    const int pos = positions[t], slot = token_slot[t];
    const int kv_begin = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float* qs = qs_all + warp * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = ldf(q + ((long long)t * heads + h) * hd + d);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;

    for (int p0 = kv_begin; p0 <= pos; p0 += 32) {
        const int p = p0 + lane;
        float s = -INFINITY;
        if (p <= pos) {
            const T* kr = pool + kv.row(slot, p, kh);
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], ldf(kr + d), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        const float pj = (p <= pos) ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= corr;
        const int cnt = min(32, pos - p0 + 1);
        for (int j = 0; j < cnt; ++j) {
            const float w = __shfl_sync(0xffffffffu, pj, j);
            const T* vr = pool + kv.v_row(slot, p0 + j, kh);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = lane + 32 * i;
                if (d < vd) acc[i] = fmaf(w, ldf(vr + d), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = lane + 32 * i;
        if (d < vd) stf(out + ((long long)t * heads + h) * vd + d, acc[i] * inv);
    }
}

// ---------------------------------------------------------------------------
// y += x (float), for parts that hand back a plain tensor.
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ y, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += ldf(y + i);
}

template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) stf(out + i, ldf(in + i));
}

}  // namespace axon

using namespace axon;


AXON_API const char* axon_last_error() { return g_error; }

// dtype codes shared with the Python side
enum { AXON_F32 = 0, AXON_BF16 = 1 };

AXON_API int axon_embed(const int32_t* tokens, const void* table, int table_dtype, float* x, int n,
                        int dim, float scale, cudaStream_t stream) {
    if (n <= 0) return AXON_OK;
    const int threads = dim >= 1024 ? 256 : 128;
    if (table_dtype == AXON_F32)
        launch_pdl(embed_kernel<float>, dim3(n), dim3(threads), 0, stream, tokens, (const float*)table, x, dim, scale);
    else if (table_dtype == AXON_BF16)
        launch_pdl(embed_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table, x, dim, scale);
    else { set_error("axon_embed: unknown table dtype %d", table_dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_embed");
}

static int rmsnorm_launch(float* x, const float* gain, const int32_t* rows, void* out, int out_dtype, int n_rows,
                          int dim, float eps, int unit_offset, SplitFold fold, cudaStream_t stream) {
    if (n_rows <= 0) return AXON_OK;
    if (out_dtype != AXON_F32 && out_dtype != AXON_BF16) { set_error("axon_rmsnorm: unknown output dtype %d", out_dtype); return AXON_BAD_ARGUMENT; }
    const int n4 = dim / 4;
    if (dim % 4 == 0 && n4 <= 8 * 1024 &&
        (((uintptr_t)x | (uintptr_t)gain | (uintptr_t)out | (uintptr_t)fold.partial | (uintptr_t)fold.bias) & 15) == 0) {
        // whole float4s, at most 8 per thread: the kernel that reads the row once
        int per = (n4 + 1023) / 1024;
        // few rows: as many threads per row as there are float4s (the shortest chain); many rows:
        // four float4s per thread, so that several rows fit an SM and enough bytes are in flight
        if (n_rows > 4 * 148 && per < 4 && n4 >= 4 * 64) per = 4;
        per = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : 8;
        int threads = ((n4 + per - 1) / per + 31) / 32 * 32;
#define AXON_NORM_CASE(TO, VPT) launch_pdl(rmsnorm_vec_kernel<TO, VPT>, dim3(n_rows), dim3(threads), 0, stream, x, gain, rows, (TO*)out, dim, eps, unit_offset, fold)
#define AXON_NORM_TYPE(VPT) do { if (out_dtype == AXON_F32) AXON_NORM_CASE(float, VPT); else AXON_NORM_CASE(__nv_bfloat16, VPT); } while (0)
        if (per == 1) AXON_NORM_TYPE(1); else if (per == 2) AXON_NORM_TYPE(2); else if (per == 4) AXON_NORM_TYPE(4); else AXON_NORM_TYPE(8);
#undef AXON_NORM_TYPE
#undef AXON_NORM_CASE
        return launch_status("axon_rmsnorm");
    }
    int threads = 128;
    while (threads < 1024 && threads * 4 < dim) threads *= 2;
    if (out_dtype == AXON_F32)
        launch_pdl(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, gain, rows, (float*)out, dim, eps, unit_offset, fold);
    else if (out_dtype == AXON_BF16)
        launch_pdl(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, gain, rows, (__nv_bfloat16*)out, dim, eps, unit_offset, fold);
    else { set_error("axon_rmsnorm: unknown output dtype %d", out_dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_rmsnorm");
}

AXON_API int axon_rmsnorm(const float* x, const float* gain, const int32_t* rows, void* out,
                          int out_dtype, int n_rows, int dim, float eps, int unit_offset,
                          cudaStream_t stream) {
    return rmsnorm_launch(const_cast<float*>(x), gain, rows, out, out_dtype, n_rows, dim, eps, unit_offset,
                          SplitFold{nullptr, nullptr, 0, 0}, stream);
}

// The norm of rows that a split-K product (axon_gemm_tc_small with `defer`) still owes its
// partial sums: x[row] += the slabs in order (+ bias), written back, then normed.  With `rows`
// only the gathered rows of x are brought up to date.
AXON_API int axon_rmsnorm_fold(float* x, const float* gain, const int32_t* rows, void* out, int out_dtype,
                               int n_rows, int dim, float eps, int unit_offset, const float* partial, int splits,
                               int ntok, const float* bias, cudaStream_t stream) {
    if (partial == nullptr || splits < 1 || ntok < 1) { set_error("axon_rmsnorm_fold: no partial sums given"); return AXON_BAD_ARGUMENT; }
    if (rows == nullptr && n_rows > ntok) { set_error("axon_rmsnorm_fold: %d rows, partial sums for %d", n_rows, ntok); return AXON_BAD_ARGUMENT; }
    return rmsnorm_launch(x, gain, rows, out, out_dtype, n_rows, dim, eps, unit_offset,
                          SplitFold{partial, bias, splits, ntok}, stream);
}

// out[m][n] (= or +=) the partial sums of a deferred split-K product, for readers that cannot
// fold them themselves.  out: float (store or accumulate) or bfloat16 (store).
template <typename TO>
__global__ void fold_partials_kernel(SplitFold fold, TO* __restrict__ out, int M, int N, int ldo, int accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)M * N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / N), n = (int)(i % N);
        float v = fold.at(m, n);
        TO* o = out + (long long)m * ldo + n;
        if (accumulate) v += ldf(o);
        stf(o, v);
    }
}

AXON_API int axon_fold_partials(const float* partial, int splits, int ntok, const float* bias, void* out,
                                int out_dtype, int M, int N, int ldo, int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return AXON_OK;
    if (partial == nullptr || splits < 1 || ntok < M) { set_error("axon_fold_partials: bad partial sums (splits %d, tokens %d of %d)", splits, M, ntok); return AXON_BAD_ARGUMENT; }
    if (accumulate && out_dtype != AXON_F32) { set_error("axon_fold_partials: the residual is float"); return AXON_BAD_ARGUMENT; }
    const SplitFold fold{partial, bias, splits, ntok};
    const long long total = (long long)M * N;
    const unsigned blocks = (unsigned)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256);
    if (out_dtype == AXON_F32) launch_pdl(fold_partials_kernel<float>, dim3(blocks), dim3(256), 0, stream, fold, (float*)out, M, N, ldo, accumulate);
    else if (out_dtype == AXON_BF16) launch_pdl(fold_partials_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, fold, (__nv_bfloat16*)out, M, N, ldo, accumulate);
    else { set_error("axon_fold_partials: unknown dtype %d", out_dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_fold_partials");
}

template <typename TA, typename TW>
static int gemm_plain_out(const void* a, const void* w, const float* bias, void* out, int out_dtype,
                          int M, int N, int K, int lda, int ldo, int mode, cudaStream_t stream) {
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (out_dtype == AXON_F32)
        gemm_plain_kernel<TA, TW, float><<<grid, 256, 0, stream>>>((const TA*)a, (const TW*)w, bias, (float*)out, M, N, K, lda, ldo, mode);
    else if (out_dtype == AXON_BF16)
        gemm_plain_kernel<TA, TW, __nv_bfloat16><<<grid, 256, 0, stream>>>((const TA*)a, (const TW*)w, bias, (__nv_bfloat16*)out, M, N, K, lda, ldo, mode);
    else { set_error("axon_gemm_plain: unknown output dtype %d", out_dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_gemm_plain");
}

// out = a . w^T (+ bias), mode 0 store / 1 add into out.  Any sizes.
AXON_API int axon_gemm_plain(const void* a, int a_dtype, const void* w, int w_dtype, const float* bias,
                             void* out, int out_dtype, int M, int N, int K, int lda, int ldo, int mode,
                             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return AXON_OK;
    if (K <= 0 || lda < K || ldo < N) { set_error("axon_gemm_plain: bad sizes M %d N %d K %d lda %d ldo %d", M, N, K, lda, ldo); return AXON_BAD_ARGUMENT; }
    if (mode == 1 && out_dtype != AXON_F32) { set_error("axon_gemm_plain: the residual is float"); return AXON_BAD_ARGUMENT; }
    if (a_dtype == AXON_F32 && w_dtype == AXON_F32) return gemm_plain_out<float, float>(a, w, bias, out, out_dtype, M, N, K, lda, ldo, mode, stream);
    if (a_dtype == AXON_BF16 && w_dtype == AXON_BF16) return gemm_plain_out<__nv_bfloat16, __nv_bfloat16>(a, w, bias, out, out_dtype, M, N, K, lda, ldo, mode, stream);
    if (a_dtype == AXON_BF16 && w_dtype == AXON_F32) return gemm_plain_out<__nv_bfloat16, float>(a, w, bias, out, out_dtype, M, N, K, lda, ldo, mode, stream);
    if (a_dtype == AXON_F32 && w_dtype == AXON_BF16) return gemm_plain_out<float, __nv_bfloat16>(a, w, bias, out, out_dtype, M, N, K, lda, ldo, mode, stream);
    set_error("axon_gemm_plain: unknown dtypes %d %d", a_dtype, w_dtype);
    return AXON_BAD_ARGUMENT;
}

AXON_API int axon_swiglu(const float* gate_up, void* act, int act_dtype, int n, int ffn, cudaStream_t stream) {
    const long long total = (long long)n * ffn;
    if (total <= 0) return AXON_OK;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (act_dtype == AXON_F32) swiglu_kernel<float><<<blocks, 256, 0, stream>>>(gate_up, (float*)act, total, ffn);
    else if (act_dtype == AXON_BF16) swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(gate_up, (__nv_bfloat16*)act, total, ffn);
    else { set_error("axon_swiglu: unknown dtype %d", act_dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_swiglu");
}

AXON_API int axon_rope_table(const int32_t* positions, const double* inv_freq, float* table, int n,
                             int half, float magnitude, cudaStream_t stream) {
    if (n <= 0 || half <= 0) return AXON_OK;
    const int total = n * half;
    launch_pdl(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, positions, inv_freq, (float2*)table, n, half, magnitude);
    return launch_status("axon_rope_table");
}

AXON_API int axon_rope_kv_write(const float* qkv, const float* table, const int32_t* positions,
                                const int32_t* token_slot, void* q_out, void* pool, int dtype,
                                const AxonKvLayout* layout, int n, int heads, int rot, int adjacent,
                                int write_kv, const float* partial, int splits, int ntok, const float* bias,
                                cudaStream_t stream) {
    // partial != null: qkv is still owed the partial sums of a deferred split-K product
    // (see axon_gemm_tc_small); they are folded here and `qkv` itself is not read
    if (n <= 0) return AXON_OK;
    if (partial != nullptr && (splits < 1 || ntok < n)) { set_error("axon_rope_kv_write: bad partial sums (splits %d, tokens %d of %d)", splits, n, ntok); return AXON_BAD_ARGUMENT; }
    const SplitFold fold{partial, partial ? bias : nullptr, splits, ntok};
    const int hd = layout->head_dim;
    if (hd % 2 || rot % 2 || rot > hd || rot < 0) { set_error("axon_rope_kv_write: head size %d / rotated size %d must be even and rot <= head", hd, rot); return AXON_BAD_ARGUMENT; }
    PagedKv kv = to_paged(layout);
    if (kv.planes == 2 && kv.v_dim % 2) { set_error("axon_rope_kv_write: value rows of %d elements are not even", kv.v_dim); return AXON_BAD_ARGUMENT; }
    if (table != nullptr && !adjacent && rot == hd && hd % 8 == 0 && kv.planes == 2 && kv.v_dim == hd &&
        (((uintptr_t)qkv | (uintptr_t)table | (uintptr_t)q_out | (uintptr_t)pool | (uintptr_t)partial | (uintptr_t)bias) & 15) == 0 &&
        (layout->page_stride * (dtype == AXON_F32 ? 4 : 2)) % 16 == 0 && (layout->entry_offset * (dtype == AXON_F32 ? 4 : 2)) % 16 == 0 &&
        (layout->v_offset * (dtype == AXON_F32 ? 4 : 2)) % 16 == 0) {
        const int quads = (heads + 2 * layout->kv_heads) * (hd / 8);
        dim3 vgrid(n, (quads + 255) / 256 > 8 ? 8 : (quads + 255) / 256);
        if (dtype == AXON_F32)
            launch_pdl(rope_kv_write_vec_kernel<float>, vgrid, dim3(256), 0, stream, qkv, (const float2*)table, positions, token_slot, (float*)q_out, (float*)pool, kv, heads, write_kv, fold);
        else if (dtype == AXON_BF16)
            launch_pdl(rope_kv_write_vec_kernel<__nv_bfloat16>, vgrid, dim3(256), 0, stream, qkv, (const float2*)table, positions, token_slot, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, kv, heads, write_kv, fold);
        else { set_error("axon_rope_kv_write: unknown dtype %d", dtype); return AXON_BAD_ARGUMENT; }
        return launch_status("axon_rope_kv_write");
    }
    const int items = (heads + layout->kv_heads) * (hd / 2) + (kv.planes == 2 ? layout->kv_heads * (kv.v_dim / 2) : 0);
    dim3 grid(n, (items + 255) / 256 > 8 ? 8 : (items + 255) / 256);
    if (dtype == AXON_F32)
        launch_pdl(rope_kv_write_kernel<float>, grid, dim3(256), 0, stream, qkv, (const float2*)table, positions, token_slot, (float*)q_out, (float*)pool, kv, heads, rot, adjacent, write_kv, fold);
    else if (dtype == AXON_BF16)
        launch_pdl(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, qkv, (const float2*)table, positions, token_slot, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, kv, heads, rot, adjacent, write_kv, fold);
    else { set_error("axon_rope_kv_write: unknown dtype %d", dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_rope_kv_write");
}

AXON_API int axon_attention_plain(const void* q, const void* pool, int dtype, const int32_t* positions,
                                  const int32_t* token_slot, void* out, const AxonKvLayout* layout,
                                  int n, int heads, float scale, int window, cudaStream_t stream) {
    if (n <= 0) return AXON_OK;
    const int hd = layout->head_dim;
    if (hd > 256 || hd < 1) { set_error("axon_attention_plain: head size %d is not in 1..256", hd); return AXON_BAD_ARGUMENT; }
    if (layout->v_dim > 256) { set_error("axon_attention_plain: value rows of %d elements exceed 256", layout->v_dim); return AXON_BAD_ARGUMENT; }
    if (heads % layout->kv_heads) { set_error("axon_attention_plain: %d heads over %d kv heads", heads, layout->kv_heads); return AXON_BAD_ARGUMENT; }
    const int warps = 4;
    const long long items = (long long)n * heads;
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * hd * sizeof(float);
    PagedKv kv = to_paged(layout);
    if (dtype == AXON_F32)
        attention_plain_kernel<float><<<blocks, warps * 32, smem, stream>>>((const float*)q, (const float*)pool, positions, token_slot, (float*)out, kv, n, heads, scale, window);
    else if (dtype == AXON_BF16)
        attention_plain_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)pool, positions, token_slot, (__nv_bfloat16*)out, kv, n, heads, scale, window);
    else { set_error("axon_attention_plain: unknown dtype %d", dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_attention_plain");
}

AXON_API int axon_residual_add(float* x, const void* y, int y_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return AXON_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (y_dtype == AXON_F32) residual_add_kernel<float><<<blocks, 256, 0, stream>>>(x, (const float*)y, n);
    else if (y_dtype == AXON_BF16) residual_add_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(x, (const __nv_bfloat16*)y, n);
    else { set_error("axon_residual_add: unknown dtype %d", y_dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_residual_add");
}

AXON_API int axon_convert(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return AXON_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == AXON_F32 && out_dtype == AXON_BF16) convert_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, n);
    else if (in_dtype == AXON_BF16 && out_dtype == AXON_F32) convert_kernel<__nv_bfloat16, float><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, n);
    else if (in_dtype == AXON_F32 && out_dtype == AXON_F32) convert_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)in, (float*)out, n);
    else if (in_dtype == AXON_BF16 && out_dtype == AXON_BF16) convert_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, n);
    else { set_error("axon_convert: unknown dtypes %d %d", in_dtype, out_dtype); return AXON_BAD_ARGUMENT; }
    return launch_status("axon_convert");
}
