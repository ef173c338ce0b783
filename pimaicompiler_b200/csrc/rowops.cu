// Row-wise glue operators of the decode path, fp16 storage / fp32 arithmetic: softmax and log_softmax over the last
// dimension, arg max over the last dimension, layer normalisation over the last dimension, tanh and masked_fill.
//
// They stand where the reference's executors forward to libtorch one tensor op at a time
// (runtime/source/executor/op_executor/aten_ops_executor.cpp: executeAtenSoftmax 3402-3436, executeAtenLogSoftmax
// 2092-2133, executeAtenArgmax 520-547, executeAtenLayerNorm 1898-1942, executeAtenTanh 3555-3568,
// executeAtenMaskedFill 2432-2467).  All are small and latency-bound at decode sizes (a 29..32320-wide logit row, a
// handful of attention scores, a 512-wide model vector): one CTA per row (128 threads, 1024 for rows of 4096 elements
// or more), the row is read with 128-bit loads when its address and length allow, reductions run in fp32 through warp
// shuffles and one shared-memory hop.
#include <math_constants.h>

#include "common.cuh"

using namespace pimb200;

namespace {

constexpr int kWideRow = 4096;   // rows at least this long get a 1024-thread CTA

template <int T>
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();   // red may still be read from the previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < T / 32; ++w) r = fmaxf(r, red[w]);
    return r;
}
template <int T>
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < T / 32; ++w) r += red[w];   // fixed order: the result does not depend on timing
    return r;
}

// element access: VEC = 8 halves per 16-byte load when the row allows it, else scalar
template <int T, bool VEC, typename F>
__device__ __forceinline__ void for_each(const __half* row, long cols, F f) {
    if (VEC) {
        const uint4* r4 = reinterpret_cast<const uint4*>(row);
        for (long c = threadIdx.x; c < (cols >> 3); c += T) {
            float xf[8];
            widen8(r4[c], xf);
#pragma unroll
            for (int j = 0; j < 8; ++j) f(c * 8 + j, xf[j]);
        }
    } else {
        for (long c = threadIdx.x; c < cols; c += T) f(c, __half2float(row[c]));
    }
}

// out[c] = g(c, row[c]) for the whole row; in the vector case eight results leave as one 16-byte store
template <int T, bool VEC, typename G>
__device__ __forceinline__ void map_store(const __half* row, __half* out, long cols, G g) {
    if (VEC) {
        const uint4* r4 = reinterpret_cast<const uint4*>(row);
        uint4* o4 = reinterpret_cast<uint4*>(out);
        for (long c = threadIdx.x; c < (cols >> 3); c += T) {
            float xf[8];
            widen8(r4[c], xf);
            __half2 h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(g(c * 8 + 2 * j, xf[2 * j]), g(c * 8 + 2 * j + 1, xf[2 * j + 1]));
            uint4 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&h[0]);
            pk.y = *reinterpret_cast<uint32_t*>(&h[1]);
            pk.z = *reinterpret_cast<uint32_t*>(&h[2]);
            pk.w = *reinterpret_cast<uint32_t*>(&h[3]);
            o4[c] = pk;
        }
    } else {
        for (long c = threadIdx.x; c < cols; c += T) out[c] = __float2half_rn(g(c, __half2float(row[c])));
    }
}

template <int T, bool VEC, bool LOG>
__global__ void __launch_bounds__(T) softmax_rows_kernel(const __half* __restrict__ x, __half* __restrict__ y,
                                                                   long cols) {
    __shared__ float red[T / 32];
    const __half* row = x + (size_t)blockIdx.x * cols;
    __half* out = y + (size_t)blockIdx.x * cols;
    float m = -CUDART_INF_F;
    for_each<T, VEC>(row, cols, [&](long, float v) { m = fmaxf(m, v); });
    m = block_max<T>(m, red);
    float s = 0.f;
    for_each<T, VEC>(row, cols, [&](long, float v) { s += expf(v - m); });
    s = block_sum<T>(s, red);
    const float inv = 1.0f / s, ls = logf(s);
    map_store<T, VEC>(row, out, cols, [&](long, float v) { return LOG ? (v - m) - ls : expf(v - m) * inv; });
}

template <int T, bool VEC>
__global__ void __launch_bounds__(T) argmax_rows_kernel(const __half* __restrict__ x, long long* __restrict__ idx,
                                                                  long cols) {
    __shared__ float red_v[T / 32];
    __shared__ long long red_i[T / 32];
    const __half* row = x + (size_t)blockIdx.x * cols;
    float bv = -CUDART_INF_F;
    long long bi = cols;   // lowest index among equal maxima wins, as in at::argmax on a contiguous row
    for_each<T, VEC>(row, cols, [&](long c, float v) {
        if (v > bv || (v == bv && c < bi)) { bv = v; bi = c; }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red_v[warp] = bv; red_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < T / 32; ++w)
            if (red_v[w] > bv || (red_v[w] == bv && red_i[w] < bi)) { bv = red_v[w]; bi = red_i[w]; }
        idx[blockIdx.x] = bi < cols ? bi : 0;   // a row of NaNs / -inf only: index 0
    }
}

// The k largest (or smallest) elements of every row, in order, with their indices: k rounds over the row (it stays in
// L1 / L2), each round the block-wide best element that comes after the previous pick in the total order
// (value, then lower index first), so no set of taken indices has to be kept.  One CTA per row.
template <int T>
__global__ void __launch_bounds__(T) topk_rows_kernel(const __half* __restrict__ x, __half* __restrict__ values,
                                                      long long* __restrict__ idx, long cols, int k, int largest) {
    __shared__ float red_v[T / 32];
    __shared__ long long red_i[T / 32];
    __shared__ float pick_v;
    __shared__ long long pick_i;
    const __half* row = x + (size_t)blockIdx.x * cols;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float sgn = largest ? 1.f : -1.f;          // smallest-first is largest-first of the negated row
    float prev_v = CUDART_INF_F;
    long long prev_i = -1;
    for (int r = 0; r < k; ++r) {
        float bv = -CUDART_INF_F;
        long long bi = cols;
        for (long c = threadIdx.x; c < cols; c += T) {
            const float v = sgn * __half2float(row[c]);
            const bool after_prev = v < prev_v || (v == prev_v && c > prev_i);
            if (after_prev && (v > bv || (v == bv && c < bi))) { bv = v; bi = c; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { red_v[warp] = bv; red_i[warp] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < T / 32; ++w)
                if (red_v[w] > bv || (red_v[w] == bv && red_i[w] < bi)) { bv = red_v[w]; bi = red_i[w]; }
            pick_v = bv;
            pick_i = bi;
            const long long out_i = bi < cols ? bi : 0;          // fewer than k comparable elements (NaNs): index 0
            values[(size_t)blockIdx.x * k + r] = row[out_i];
            idx[(size_t)blockIdx.x * k + r] = out_i;
        }
        __syncthreads();
        prev_v = pick_v;
        prev_i = pick_i;
    }
}

template <int T, bool VEC>
__global__ void __launch_bounds__(T) layer_norm_rows_kernel(const __half* __restrict__ x,
                                                                      const __half* __restrict__ gamma,
                                                                      const __half* __restrict__ beta,
                                                                      __half* __restrict__ y, long cols, float eps) {
    __shared__ float red[T / 32];
    const __half* row = x + (size_t)blockIdx.x * cols;
    __half* out = y + (size_t)blockIdx.x * cols;
    float s = 0.f;
    for_each<T, VEC>(row, cols, [&](long, float v) { s += v; });
    const float mean = block_sum<T>(s, red) / (float)cols;
    float q = 0.f;
    for_each<T, VEC>(row, cols, [&](long, float v) { const float d = v - mean; q += d * d; });
    const float rstd = rsqrtf(block_sum<T>(q, red) / (float)cols + eps);   // biased variance, as at::layer_norm
    map_store<T, VEC>(row, out, cols, [&](long c, float v) {
        float r = (v - mean) * rstd;
        if (gamma) r *= __half2float(gamma[c]);
        if (beta) r += __half2float(beta[c]);
        return r;
    });
}

__global__ void tanh_f16_kernel(const __half* __restrict__ x, __half* __restrict__ y, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = __float2half_rn(tanhf(__half2float(x[i])));
}

__global__ void masked_fill_f16_kernel(const __half* __restrict__ x, const unsigned char* __restrict__ mask, __half value,
                                       __half* __restrict__ y, size_t n, size_t mask_n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = mask[i % mask_n] ? value : x[i];
}

// out[i, :] = table[idx[i], :], rows of row_bytes bytes; an index outside [0, n_table) yields a zero row
__global__ void gather_rows_kernel(const unsigned char* __restrict__ table, const long long* __restrict__ idx,
                                   unsigned char* __restrict__ out, size_t row_bytes, long n_table, int vec16) {
    const long long r = idx[blockIdx.x];
    const bool ok = r >= 0 && r < n_table;
    const unsigned char* src = table + (size_t)(ok ? r : 0) * row_bytes;
    unsigned char* dst = out + (size_t)blockIdx.x * row_bytes;
    if (vec16) {
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        for (size_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = ok ? reinterpret_cast<const uint4*>(src)[i] : zero;
    } else {
        for (size_t i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = ok ? src[i] : (unsigned char)0;
    }
}

// table[idx[i], :] = src[i, :]: the write-side twin of the gather (a KV-cache append at a position that lives on the
// device); an index outside [0, n_table) is skipped
__global__ void scatter_rows_kernel(unsigned char* __restrict__ table, const long long* __restrict__ idx,
                                    const unsigned char* __restrict__ src, size_t row_bytes, long n_table, int vec16) {
    const long long r = idx[blockIdx.x];
    if (r < 0 || r >= n_table) return;
    unsigned char* dst = table + (size_t)r * row_bytes;
    const unsigned char* s = src + (size_t)blockIdx.x * row_bytes;
    if (vec16) {
        for (size_t i = threadIdx.x; i < row_bytes / 16; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(s)[i];
    } else {
        for (size_t i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = s[i];
    }
}

// Single-query (decode-step) multi-head attention over a key / value cache: one CTA per head,
//     out[h] = softmax(scale * q[h] . K[0..L)[h]^T) . V[0..L)[h],   L = *len_dev + len_add (or len_add when len_dev is NULL).
// Scores live in shared memory (fp32), so L is limited by kAttnMaxLen.  Rows of K / V are kv_stride elements apart.
constexpr int kAttnThreads = 128;
constexpr int kAttnMaxLen = 8192;

__global__ void __launch_bounds__(kAttnThreads) attention_row_kernel(const __half* __restrict__ q, const __half* __restrict__ K,
                                                                     const __half* __restrict__ V, const long long* len_dev,
                                                                     long len_add, long max_len, __half* __restrict__ out,
                                                                     int hd, long kv_stride, float scale) {
    extern __shared__ float sc[];            // [L] scores, then [kAttnThreads / 32][hd] partial outputs
    __shared__ float red[kAttnThreads / 32];
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long L = (len_dev ? (long)*len_dev : 0) + len_add;
    L = L < 0 ? 0 : (L > max_len ? max_len : L);
    const __half* qh = q + (size_t)h * hd;
    // scores: a warp per cache row, lanes along the head dimension
    for (long t = warp; t < L; t += kAttnThreads / 32) {
        const __half* kr = K + (size_t)t * kv_stride + (size_t)h * hd;
        float a = 0.f;
        for (int j = lane; j < hd; j += 32) a = fmaf(__half2float(qh[j]), __half2float(kr[j]), a);
        a = warp_sum(a);
        if (lane == 0) sc[t] = a * scale;
    }
    __syncthreads();
    float m = -CUDART_INF_F;
    for (long t = threadIdx.x; t < L; t += kAttnThreads) m = fmaxf(m, sc[t]);
    m = block_max<kAttnThreads>(m, red);
    float s = 0.f;
    for (long t = threadIdx.x; t < L; t += kAttnThreads) {
        const float e = expf(sc[t] - m);
        sc[t] = e;
        s += e;
    }
    s = block_sum<kAttnThreads>(s, red);   // ends with a barrier: every sc[t] is final
    const float inv = L > 0 ? 1.0f / s : 0.f;
    // weighted sum: warp w takes rows w, w+4, ...; lanes along the head dimension; partials meet in shared memory
    float* part = sc + max_len;
    for (int j = lane; j < hd; j += 32) {
        float a = 0.f;
        for (long t = warp; t < L; t += kAttnThreads / 32)
            a = fmaf(sc[t], __half2float(V[(size_t)t * kv_stride + (size_t)h * hd + j]), a);
        part[warp * hd + j] = a;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < hd; j += kAttnThreads) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnThreads / 32; ++w) a += part[w * hd + j];
        out[(size_t)h * hd + j] = __float2half_rn(a * inv);
    }
}

// Batched form of attention_row_kernel: blockIdx.y is the sequence; every sequence has its own cache (seq_stride
// elements after the previous one) and its own length (len_dev[seq * len_inc]).
__global__ void __launch_bounds__(kAttnThreads) attention_rows_kernel(const __half* __restrict__ q, const __half* __restrict__ K,
                                                                      const __half* __restrict__ V, const long long* len_dev,
                                                                      long len_inc, long len_add, long max_len,
                                                                      __half* __restrict__ out, int hd, long kv_stride,
                                                                      long seq_stride, long q_stride, long out_stride,
                                                                      float scale) {
    extern __shared__ float sc[];            // [max_len] scores, then [kAttnThreads / 32][hd] partial outputs
    __shared__ float red[kAttnThreads / 32];
    const int h = blockIdx.x, seq = blockIdx.y, heads = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long L = (len_dev ? (long)len_dev[(size_t)seq * len_inc] : 0) + len_add;
    L = L < 0 ? 0 : (L > max_len ? max_len : L);
    (void)heads;
    const __half* qh = q + (size_t)seq * q_stride + (size_t)h * hd;
    const __half* Ks = K + (size_t)seq * seq_stride + (size_t)h * hd;
    const __half* Vs = V + (size_t)seq * seq_stride + (size_t)h * hd;
    for (long t = warp; t < L; t += kAttnThreads / 32) {
        const __half* kr = Ks + (size_t)t * kv_stride;
        float a = 0.f;
        for (int j = lane; j < hd; j += 32) a = fmaf(__half2float(qh[j]), __half2float(kr[j]), a);
        a = warp_sum(a);
        if (lane == 0) sc[t] = a * scale;
    }
    __syncthreads();
    float m = -CUDART_INF_F;
    for (long t = threadIdx.x; t < L; t += kAttnThreads) m = fmaxf(m, sc[t]);
    m = block_max<kAttnThreads>(m, red);
    float s = 0.f;
    for (long t = threadIdx.x; t < L; t += kAttnThreads) {
        const float e = expf(sc[t] - m);
        sc[t] = e;
        s += e;
    }
    s = block_sum<kAttnThreads>(s, red);   // ends with a barrier: every sc[t] is final
    const float inv = L > 0 ? 1.0f / s : 0.f;
    float* part = sc + max_len;
    for (int j = lane; j < hd; j += 32) {
        float a = 0.f;
        for (long t = warp; t < L; t += kAttnThreads / 32) a = fmaf(sc[t], __half2float(Vs[(size_t)t * kv_stride + j]), a);
        part[warp * hd + j] = a;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < hd; j += kAttnThreads) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnThreads / 32; ++w) a += part[w * hd + j];
        out[(size_t)seq * out_stride + (size_t)h * hd + j] = __float2half_rn(a * inv);
    }
}

// The same batched single-query attention with a WARP per (head, sequence), for head widths of 64 or 128 and up to 128
// cache rows: lanes along the cache rows for the scores (each lane reads whole 128- or 256-byte key rows, the query comes
// from shared memory as a broadcast), warp shuffles for the softmax, lanes along the head dimension for the weighted sum
// (one coalesced row of V per cache row, eight rows of loads in flight).  No block-wide barrier, nothing serial per row.
constexpr int kWarpAttnWarps = 8;
constexpr int kWarpAttnMaxLen = 128;

template <int EPL>   // elements of the head dimension per lane: 2 (head_dim 64) or 4 (head_dim 128)
__global__ void __launch_bounds__(kWarpAttnWarps * 32) attention_rows_warp_kernel(
    const __half* __restrict__ q, const __half* __restrict__ K, const __half* __restrict__ V, const long long* len_dev,
    long len_inc, long len_add, long max_len, __half* __restrict__ out, int heads, int n_seq, long kv_stride, long seq_stride,
    long q_stride, long out_stride, float scale) {
    constexpr int HD = EPL * 32;
    constexpr int KPL = kWarpAttnMaxLen / 32;     // cache rows per lane
    __shared__ __align__(16) float qs[kWarpAttnWarps][HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long task = (long)blockIdx.x * kWarpAttnWarps + warp;   // head fastest: the heads of a sequence share cache lines
    if (task >= (long)heads * n_seq) return;
    const int h = (int)(task % heads), seq = (int)(task / heads);
    long L = (len_dev ? (long)len_dev[(size_t)seq * len_inc] : 0) + len_add;
    L = L < 0 ? 0 : (L > max_len ? max_len : L);
    const __half* qh = q + (size_t)seq * q_stride + (size_t)h * HD;
    const __half* Ks = K + (size_t)seq * seq_stride + (size_t)h * HD;
    const __half* Vs = V + (size_t)seq * seq_stride + (size_t)h * HD;
#pragma unroll
    for (int e = 0; e < EPL; ++e) qs[warp][lane * EPL + e] = __half2float(qh[lane * EPL + e]) * scale;
    __syncwarp();
    float sc[KPL];
    float m = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
        const long t = lane + 32 * i;
        sc[i] = -CUDART_INF_F;
        if (t < L) {
            const uint4* kr = reinterpret_cast<const uint4*>(Ks + (size_t)t * kv_stride);
            float a = 0.f;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                float kf[8];
                widen8(__ldg(kr + c), kf);
                const float4 q0 = *reinterpret_cast<const float4*>(&qs[warp][c * 8]);
                const float4 q1 = *reinterpret_cast<const float4*>(&qs[warp][c * 8 + 4]);
                a = fmaf(q0.x, kf[0], a); a = fmaf(q0.y, kf[1], a); a = fmaf(q0.z, kf[2], a); a = fmaf(q0.w, kf[3], a);
                a = fmaf(q1.x, kf[4], a); a = fmaf(q1.y, kf[5], a); a = fmaf(q1.z, kf[6], a); a = fmaf(q1.w, kf[7], a);
            }
            sc[i] = a;
            m = fmaxf(m, a);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
        sc[i] = (lane + 32 * i < L) ? expf(sc[i] - m) : 0.f;
        sum += sc[i];
    }
    sum = warp_sum(sum);
    float acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;
    const __half* vcol = Vs + lane * EPL;
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
        if ((long)32 * i >= L) break;
        const int rows = (int)min((long)32, L - 32 * i);
        for (int t0 = 0; t0 < rows; t0 += 8) {
            float vf[8][EPL];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const long t = 32 * i + min(t0 + u, rows - 1);       // the tail repeats the last row with weight 0
                if (EPL == 2) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(vcol + (size_t)t * kv_stride));
                    vf[u][0] = f.x; vf[u][1] = f.y;
                } else {
                    const uint2 raw = *reinterpret_cast<const uint2*>(vcol + (size_t)t * kv_stride);
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                    vf[u][0] = f0.x; vf[u][1] = f0.y; vf[u][EPL - 2] = f1.x; vf[u][EPL - 1] = f1.y;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                float p = __shfl_sync(0xffffffffu, sc[i], (t0 + u) & 31);
                if (t0 + u >= rows) p = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[e] = fmaf(p, vf[u][e], acc[e]);
            }
        }
    }
    const float inv = L > 0 ? 1.0f / sum : 0.f;
    __half* o = out + (size_t)seq * out_stride + (size_t)h * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] = __float2half_rn(acc[e] * inv);
}

// Additive (normalised Bahdanau) attention of a decode step:
//     e[s]   = sum_h v[h] * tanh(keys_proj[s, h] + q[h] + bias[h]),  s < length
//     ctx[h] = sum_s softmax(e)[s] * values[s, h]
// Row s of sentence j lies at j * seq_stride + s * row_stride elements (time-major encoder output: row_stride =
// sentences * H, seq_stride = H).  Two launches, both with far more CTAs than SMs, because one CTA per sentence walks
// its 50 rows one dependent load after the other: (1) a warp per (sentence, source position) computes the score,
// (2) a CTA per (sentence, slice of H) turns the sentence's scores into weights and accumulates its slice of the
// context, eight rows of loads in flight per thread.
constexpr int kAddAttnThreads = 256;
constexpr int kAddAttnSlice = 256;       // context elements per CTA of the second launch (two per thread, 128 threads)

__global__ void __launch_bounds__(kAddAttnThreads) additive_scores_kernel(
    const __half* __restrict__ q, const __half* __restrict__ keys_proj, const long long* __restrict__ lengths,
    const __half* __restrict__ v, const __half* __restrict__ bias, float* __restrict__ scores, int n_seq, long max_len,
    int H, long row_stride, long seq_stride) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long row = (long)blockIdx.x * (kAddAttnThreads / 32) + warp;     // (sentence, position), position fastest
    if (row >= (long)n_seq * max_len) return;
    const int seq = (int)(row / max_len);
    const long s = row % max_len;
    long L = lengths ? (long)lengths[seq] : max_len;
    L = L < 0 ? 0 : (L > max_len ? max_len : L);
    if (s >= L) return;
    const __half* kr = keys_proj + (size_t)seq * seq_stride + (size_t)s * row_stride;
    const __half* qr = q + (size_t)seq * H;
    float a = 0.f;
    const bool vec = (H % 8 == 0) && (row_stride % 8 == 0) && (seq_stride % 8 == 0) &&
                     ((reinterpret_cast<uintptr_t>(keys_proj) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(q) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(v) & 15u) == 0) && (!bias || (reinterpret_cast<uintptr_t>(bias) & 15u) == 0);
    if (vec) {
        for (int c = lane; c < (H >> 3); c += 32) {
            float kf[8], qf[8], vf[8], bf[8];
            widen8(__ldg(reinterpret_cast<const uint4*>(kr) + c), kf);
            widen8(__ldg(reinterpret_cast<const uint4*>(qr) + c), qf);
            widen8(__ldg(reinterpret_cast<const uint4*>(v) + c), vf);
            if (bias) widen8(__ldg(reinterpret_cast<const uint4*>(bias) + c), bf);
#pragma unroll
            for (int i = 0; i < 8; ++i) a = fmaf(vf[i], tanhf_(kf[i] + (qf[i] + (bias ? bf[i] : 0.f))), a);
        }
    } else {
        for (int h = lane; h < H; h += 32)
            a = fmaf(__half2float(v[h]),
                     tanhf_(__half2float(kr[h]) + (__half2float(qr[h]) + (bias ? __half2float(bias[h]) : 0.f))), a);
    }
    a = warp_sum(a);
    if (lane == 0) scores[row] = a;
}

__global__ void __launch_bounds__(kAddAttnSlice / 2) additive_context_kernel(
    const float* __restrict__ scores, const __half* __restrict__ values, const long long* __restrict__ lengths,
    __half* __restrict__ ctx, long max_len, int H, long row_stride, long seq_stride, long ctx_stride) {
    extern __shared__ float sc[];            // [max_len] softmax weights of this sentence
    __shared__ float red[kAddAttnSlice / 64];
    constexpr int T = kAddAttnSlice / 2;
    const int seq = blockIdx.y;
    long L = lengths ? (long)lengths[seq] : max_len;
    L = L < 0 ? 0 : (L > max_len ? max_len : L);
    float m = -CUDART_INF_F;
    for (long s = threadIdx.x; s < L; s += T) m = fmaxf(m, scores[(size_t)seq * max_len + s]);
    m = block_max<T>(m, red);
    float sum = 0.f;
    for (long s = threadIdx.x; s < L; s += T) {
        const float e = expf(scores[(size_t)seq * max_len + s] - m);
        sc[s] = e;
        sum += e;
    }
    sum = block_sum<T>(sum, red);             // ends with a barrier: every sc[s] is final
    const float inv = L > 0 ? 1.0f / sum : 0.f;
    const int h = blockIdx.x * kAddAttnSlice + threadIdx.x * 2;
    if (h >= H) return;
    const __half* vals = values + (size_t)seq * seq_stride + h;
    __half* out = ctx + (size_t)seq * ctx_stride + h;
    if (h + 1 < H && (row_stride % 2 == 0) && (seq_stride % 2 == 0) && (ctx_stride % 2 == 0) &&
        ((reinterpret_cast<uintptr_t>(values) & 3u) == 0) && ((reinterpret_cast<uintptr_t>(ctx) & 3u) == 0)) {
        float a0 = 0.f, a1 = 0.f;
        long s = 0;
        for (; s + 8 <= L; s += 8) {
            __half2 x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = *reinterpret_cast<const __half2*>(vals + (size_t)(s + i) * row_stride);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 f = __half22float2(x[i]);
                a0 = fmaf(sc[s + i], f.x, a0);
                a1 = fmaf(sc[s + i], f.y, a1);
            }
        }
        for (; s < L; ++s) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(vals + (size_t)s * row_stride));
            a0 = fmaf(sc[s], f.x, a0);
            a1 = fmaf(sc[s], f.y, a1);
        }
        *reinterpret_cast<__half2*>(out) = __floats2half2_rn(a0 * inv, a1 * inv);
    } else {
        for (int e = 0; e < 2 && h + e < H; ++e) {
            float a = 0.f;
            for (long s = 0; s < L; ++s) a = fmaf(sc[s], __half2float(vals[(size_t)s * row_stride + e]), a);
            out[e] = __float2half_rn(a * inv);
        }
    }
}

// y = layer_norm(x + r) per row: the residual connection and the normalisation behind every Transformer sub-layer in one
// pass (the sum lives in shared memory as fp32; each thread re-reads only the entries it wrote).
template <int T>
__global__ void __launch_bounds__(T) add_layer_norm_rows_kernel(const __half* __restrict__ x, const __half* __restrict__ r,
                                                                const __half* __restrict__ gamma, const __half* __restrict__ beta,
                                                                __half* __restrict__ y, long cols, float eps) {
    extern __shared__ float sum_row[];
    __shared__ float red[T / 32];
    const __half* xr = x + (size_t)blockIdx.x * cols;
    const __half* rr = r + (size_t)blockIdx.x * cols;
    __half* out = y + (size_t)blockIdx.x * cols;
    float s = 0.f;
    for (long c = threadIdx.x; c < cols; c += T) {
        const float v = __half2float(xr[c]) + __half2float(rr[c]);
        sum_row[c] = v;
        s += v;
    }
    const float mean = block_sum<T>(s, red) / (float)cols;
    float q = 0.f;
    for (long c = threadIdx.x; c < cols; c += T) { const float d = sum_row[c] - mean; q += d * d; }
    const float rstd = rsqrtf(block_sum<T>(q, red) / (float)cols + eps);
    for (long c = threadIdx.x; c < cols; c += T) {
        float v = (sum_row[c] - mean) * rstd;
        if (gamma) v *= __half2float(gamma[c]);
        if (beta) v += __half2float(beta[c]);
        out[c] = __float2half_rn(v);
    }
}

// Multi-head self-attention over every position of a batch of padded sequences (the encoder side of a Transformer):
// one CTA per (head, sequence) holds the sequence's keys and values of that head in shared memory; a warp per query row
// computes its scores (lanes along the keys), the softmax over the sequence's own length, and the weighted sum (lanes
// along the head dimension).  Query rows past the length give zeros.
constexpr int kBlockAttnThreads = 128;

__global__ void __launch_bounds__(kBlockAttnThreads) attention_block_kernel(
    const __half* __restrict__ Q, const __half* __restrict__ K, const __half* __restrict__ V,
    const long long* __restrict__ lengths, __half* __restrict__ out, long max_len, int hd, long row_stride, long seq_stride,
    long out_row_stride, long out_seq_stride, float scale) {
    extern __shared__ __align__(16) unsigned char blk_smem[];
    const int h = blockIdx.x, seq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kp = hd + 2;                                   // padded key row (halves): lanes on different rows, different banks
    __half* Ks = reinterpret_cast<__half*>(blk_smem);         // [max_len][kp]
    __half* Vs = Ks + (size_t)max_len * kp;                   // [max_len][hd]
    float* qs = reinterpret_cast<float*>(Vs + (size_t)max_len * hd);   // [warps][hd]
    float* ps = qs + (kBlockAttnThreads / 32) * hd;           // [warps][max_len]
    long L = lengths ? (long)lengths[seq] : max_len;
    L = L < 0 ? 0 : (L > max_len ? max_len : L);
    const size_t base = (size_t)seq * seq_stride + (size_t)h * hd;
    for (long i = threadIdx.x; i < L * hd; i += kBlockAttnThreads) {
        const long s_ = i / hd;
        const int c = (int)(i % hd);
        Ks[s_ * kp + c] = K[base + (size_t)s_ * row_stride + c];
        Vs[s_ * hd + c] = V[base + (size_t)s_ * row_stride + c];
    }
    __syncthreads();
    float* qw = qs + warp * hd;
    float* pw = ps + (size_t)warp * max_len;
    for (long qi = warp; qi < max_len; qi += kBlockAttnThreads / 32) {
        __half* o = out + (size_t)seq * out_seq_stride + (size_t)qi * out_row_stride + (size_t)h * hd;
        if (qi >= L) {
            for (int c = lane; c < hd; c += 32) o[c] = __float2half_rn(0.f);
            continue;
        }
        for (int c = lane; c < hd; c += 32) qw[c] = __half2float(Q[base + (size_t)qi * row_stride + c]) * scale;
        __syncwarp();
        float m = -CUDART_INF_F;
        for (long s_ = lane; s_ < L; s_ += 32) {
            float a = 0.f;
            for (int c = 0; c < hd; ++c) a = fmaf(qw[c], __half2float(Ks[s_ * kp + c]), a);
            pw[s_] = a;
            m = fmaxf(m, a);
        }
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o2));
        float sum = 0.f;
        for (long s_ = lane; s_ < L; s_ += 32) {
            const float e = expf(pw[s_] - m);
            pw[s_] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        __syncwarp();
        const float inv = 1.0f / sum;
        for (int c = lane; c < hd; c += 32) {
            float a = 0.f;
            for (long s_ = 0; s_ < L; ++s_) a = fmaf(pw[s_], __half2float(Vs[s_ * hd + c]), a);
            o[c] = __float2half_rn(a * inv);
        }
        __syncwarp();
    }
}

inline unsigned flat_grid(size_t n) {
    const size_t g = (n + 255) / 256;
    return (unsigned)(g > (size_t)kNumSmB200 * 8 ? (size_t)kNumSmB200 * 8 : (g ? g : 1));
}
inline bool rows_ok(long rows, long cols) { return rows > 0 && cols > 0 && rows <= 0x7fffffffL; }

}  // namespace

extern "C" int pimb200_softmax_rows(const void* x, void* y, long rows, long cols, int log_softmax, void* stream) {
    if (rows == 0 || cols == 0) return PIMB200_OK;   // empty tensors carry no storage
    if (!x || !y || !rows_ok(rows, cols)) return PIMB200_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xp = static_cast<const __half*>(x);
    __half* yp = static_cast<__half*>(y);
    const bool vec = cols % 8 == 0 && aligned16(x) && aligned16(y);
    const unsigned grid = (unsigned)rows;
    if (cols >= kWideRow) {
        if (vec) {
            if (log_softmax) softmax_rows_kernel<1024, true, true><<<grid, 1024, 0, st>>>(xp, yp, cols);
            else softmax_rows_kernel<1024, true, false><<<grid, 1024, 0, st>>>(xp, yp, cols);
        } else {
            if (log_softmax) softmax_rows_kernel<1024, false, true><<<grid, 1024, 0, st>>>(xp, yp, cols);
            else softmax_rows_kernel<1024, false, false><<<grid, 1024, 0, st>>>(xp, yp, cols);
        }
    } else if (vec) {
        if (log_softmax) softmax_rows_kernel<128, true, true><<<grid, 128, 0, st>>>(xp, yp, cols);
        else softmax_rows_kernel<128, true, false><<<grid, 128, 0, st>>>(xp, yp, cols);
    } else {
        if (log_softmax) softmax_rows_kernel<128, false, true><<<grid, 128, 0, st>>>(xp, yp, cols);
        else softmax_rows_kernel<128, false, false><<<grid, 128, 0, st>>>(xp, yp, cols);
    }
    return launch_status();
}

extern "C" int pimb200_argmax_rows(const void* x, long long* idx, long rows, long cols, void* stream) {
    if (rows == 0) return PIMB200_OK;
    if (!x || !idx || !rows_ok(rows, cols)) return PIMB200_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xp = static_cast<const __half*>(x);
    const bool vec = cols % 8 == 0 && aligned16(x);
    const unsigned grid = (unsigned)rows;
    if (cols >= kWideRow) {
        if (vec) argmax_rows_kernel<1024, true><<<grid, 1024, 0, st>>>(xp, idx, cols);
        else argmax_rows_kernel<1024, false><<<grid, 1024, 0, st>>>(xp, idx, cols);
    } else {
        if (vec) argmax_rows_kernel<128, true><<<grid, 128, 0, st>>>(xp, idx, cols);
        else argmax_rows_kernel<128, false><<<grid, 128, 0, st>>>(xp, idx, cols);
    }
    return launch_status();
}

extern "C" int pimb200_layer_norm_rows(const void* x, const void* gamma, const void* beta, void* y, long rows, long cols,
                                       float eps, void* stream) {
    if (rows == 0 || cols == 0) return PIMB200_OK;
    if (!x || !y || !rows_ok(rows, cols)) return PIMB200_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xp = static_cast<const __half*>(x);
    const __half* g = static_cast<const __half*>(gamma);
    const __half* b = static_cast<const __half*>(beta);
    __half* yp = static_cast<__half*>(y);
    const bool vec = cols % 8 == 0 && aligned16(x) && aligned16(y);
    const unsigned grid = (unsigned)rows;
    if (cols >= kWideRow) {
        if (vec) layer_norm_rows_kernel<1024, true><<<grid, 1024, 0, st>>>(xp, g, b, yp, cols, eps);
        else layer_norm_rows_kernel<1024, false><<<grid, 1024, 0, st>>>(xp, g, b, yp, cols, eps);
    } else {
        if (vec) layer_norm_rows_kernel<128, true><<<grid, 128, 0, st>>>(xp, g, b, yp, cols, eps);
        else layer_norm_rows_kernel<128, false><<<grid, 128, 0, st>>>(xp, g, b, yp, cols, eps);
    }
    return launch_status();
}

extern "C" int pimb200_tanh_f16(const void* x, void* y, size_t n, void* stream) {
    if (n == 0) return PIMB200_OK;
    if (!x || !y) return PIMB200_ERR_BAD_ARG;
    tanh_f16_kernel<<<flat_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __half*>(x),
                                                                                 static_cast<__half*>(y), n);
    return launch_status();
}

extern "C" int pimb200_masked_fill_f16(const void* x, const unsigned char* mask, float value, void* y, size_t n,
                                       size_t mask_n, void* stream) {
    if (n == 0) return PIMB200_OK;
    if (!x || !y || !mask) return PIMB200_ERR_BAD_ARG;
    if (mask_n == 0 || n % mask_n != 0) return PIMB200_ERR_BAD_ARG;
    masked_fill_f16_kernel<<<flat_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), mask, __float2half_rn(value), static_cast<__half*>(y), n, mask_n);
    return launch_status();
}

extern "C" int pimb200_gather_rows(const void* table, const long long* idx, void* out, long n_idx, size_t row_bytes,
                                   long n_table, void* stream) {
    if (n_idx == 0 || row_bytes == 0) return PIMB200_OK;
    if (!table || !idx || !out || n_idx < 0 || n_idx > 0x7fffffffL || n_table <= 0) return PIMB200_ERR_BAD_ARG;
    const int vec16 = (row_bytes % 16 == 0 && aligned16(table) && aligned16(out)) ? 1 : 0;
    gather_rows_kernel<<<(unsigned)n_idx, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const unsigned char*>(table), idx, static_cast<unsigned char*>(out), row_bytes, n_table, vec16);
    return launch_status();
}

extern "C" int pimb200_scatter_rows(void* table, const long long* idx, const void* src, long n_idx, size_t row_bytes,
                                    long n_table, void* stream) {
    if (n_idx == 0 || row_bytes == 0) return PIMB200_OK;
    if (!table || !idx || !src || n_idx < 0 || n_idx > 0x7fffffffL || n_table <= 0) return PIMB200_ERR_BAD_ARG;
    const int vec16 = (row_bytes % 16 == 0 && aligned16(table) && aligned16(src)) ? 1 : 0;
    scatter_rows_kernel<<<(unsigned)n_idx, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<unsigned char*>(table), idx, static_cast<const unsigned char*>(src), row_bytes, n_table, vec16);
    return launch_status();
}

extern "C" int pimb200_attention_row(const void* q, const void* K, const void* V, const long long* len_dev, long len_add,
                                     long max_len, void* out, int heads, int head_dim, long kv_stride, float scale,
                                     void* stream) {
    if (!q || !K || !V || !out || heads <= 0 || head_dim <= 0 || max_len <= 0 || kv_stride < (long)heads * head_dim)
        return PIMB200_ERR_BAD_ARG;
    if (max_len > kAttnMaxLen || head_dim > 1024) return PIMB200_ERR_UNSUPPORTED;
    const size_t smem = ((size_t)max_len + (size_t)(kAttnThreads / 32) * head_dim) * sizeof(float);
    // the kernel runs within the default 48 KB of shared memory per CTA (16 B of it static): larger score / partial
    // buffers are refused here instead of failing at launch
    if (smem + 16 > 48 * 1024) return PIMB200_ERR_UNSUPPORTED;
    attention_row_kernel<<<(unsigned)heads, kAttnThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(q), static_cast<const __half*>(K), static_cast<const __half*>(V), len_dev, len_add,
        max_len, static_cast<__half*>(out), head_dim, kv_stride, scale);
    return launch_status();
}

extern "C" int pimb200_attention_rows(const void* q, const void* K, const void* V, const long long* len_dev, long len_inc,
                                      long len_add, long max_len, void* out, int n_seq, int heads, int head_dim,
                                      long kv_stride, long seq_stride, long q_stride, long out_stride, float scale,
                                      void* stream) {
    if (n_seq == 0) return PIMB200_OK;
    if (!q || !K || !V || !out || n_seq < 0 || n_seq > 65535 || heads <= 0 || head_dim <= 0 || max_len <= 0 ||
        kv_stride < (long)heads * head_dim || seq_stride < 0 || len_inc < 0 || q_stride < (long)heads * head_dim ||
        out_stride < (long)heads * head_dim)
        return PIMB200_ERR_BAD_ARG;
    if (max_len > kAttnMaxLen || head_dim > 1024) return PIMB200_ERR_UNSUPPORTED;
    // a warp per (head, sequence) when the head width and the cache length allow it and every row is 16-byte aligned
    const bool rows16 = aligned16(q) && aligned16(K) && aligned16(V) && kv_stride % 8 == 0 && seq_stride % 8 == 0 && q_stride % 8 == 0;
    if ((head_dim == 64 || head_dim == 128) && max_len <= kWarpAttnMaxLen && rows16) {
        const long tasks = (long)heads * n_seq;
        const unsigned grid = (unsigned)((tasks + kWarpAttnWarps - 1) / kWarpAttnWarps);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        if (head_dim == 64)
            attention_rows_warp_kernel<2><<<grid, kWarpAttnWarps * 32, 0, st>>>(
                static_cast<const __half*>(q), static_cast<const __half*>(K), static_cast<const __half*>(V), len_dev, len_inc,
                len_add, max_len, static_cast<__half*>(out), heads, n_seq, kv_stride, seq_stride, q_stride, out_stride, scale);
        else
            attention_rows_warp_kernel<4><<<grid, kWarpAttnWarps * 32, 0, st>>>(
                static_cast<const __half*>(q), static_cast<const __half*>(K), static_cast<const __half*>(V), len_dev, len_inc,
                len_add, max_len, static_cast<__half*>(out), heads, n_seq, kv_stride, seq_stride, q_stride, out_stride, scale);
        return launch_status();
    }
    const size_t smem = ((size_t)max_len + (size_t)(kAttnThreads / 32) * head_dim) * sizeof(float);
    if (smem + 16 > 48 * 1024) return PIMB200_ERR_UNSUPPORTED;
    attention_rows_kernel<<<dim3((unsigned)heads, (unsigned)n_seq), kAttnThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(q), static_cast<const __half*>(K), static_cast<const __half*>(V), len_dev, len_inc, len_add,
        max_len, static_cast<__half*>(out), head_dim, kv_stride, seq_stride, q_stride, out_stride, scale);
    return launch_status();
}

extern "C" int pimb200_additive_attention(const void* q, const void* keys_proj, const void* values, const long long* lengths,
                                          const void* v, const void* bias, void* ctx, float* scores, int n_seq,
                                          long max_len, int H, long row_stride, long seq_stride, long ctx_stride,
                                          void* stream) {
    if (n_seq == 0) return PIMB200_OK;
    if (!q || !keys_proj || !values || !v || !ctx || !scores || n_seq < 0 || n_seq > 65535 || max_len <= 0 || H <= 0 ||
        row_stride < H || seq_stride < 0 || ctx_stride < H)
        return PIMB200_ERR_BAD_ARG;
    if ((size_t)max_len * sizeof(float) + 64 > 48 * 1024) return PIMB200_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long rows = (long)n_seq * max_len;
    additive_scores_kernel<<<(unsigned)((rows + kAddAttnThreads / 32 - 1) / (kAddAttnThreads / 32)), kAddAttnThreads, 0, st>>>(
        static_cast<const __half*>(q), static_cast<const __half*>(keys_proj), lengths, static_cast<const __half*>(v),
        static_cast<const __half*>(bias), scores, n_seq, max_len, H, row_stride, seq_stride);
    additive_context_kernel<<<dim3((unsigned)((H + kAddAttnSlice - 1) / kAddAttnSlice), (unsigned)n_seq), kAddAttnSlice / 2,
                              (size_t)max_len * sizeof(float), st>>>(
        scores, static_cast<const __half*>(values), lengths, static_cast<__half*>(ctx), max_len, H, row_stride, seq_stride,
        ctx_stride);
    return launch_status();
}

extern "C" int pimb200_add_layer_norm_rows(const void* x, const void* r, const void* gamma, const void* beta, void* y,
                                           long rows, long cols, float eps, void* stream) {
    if (rows == 0 || cols == 0) return PIMB200_OK;
    if (!x || !r || !y || !rows_ok(rows, cols)) return PIMB200_ERR_BAD_ARG;
    if ((size_t)cols * sizeof(float) + 64 > 48 * 1024) return PIMB200_ERR_UNSUPPORTED;
    add_layer_norm_rows_kernel<128><<<(unsigned)rows, 128, (size_t)cols * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(r), static_cast<const __half*>(gamma),
        static_cast<const __half*>(beta), static_cast<__half*>(y), cols, eps);
    return launch_status();
}

extern "C" int pimb200_attention_block(const void* q, const void* k, const void* v, const long long* lengths, void* out,
                                       int n_seq, long max_len, int heads, int head_dim, long row_stride, long seq_stride,
                                       long out_row_stride, long out_seq_stride, float scale, void* stream) {
    if (n_seq == 0) return PIMB200_OK;
    if (!q || !k || !v || !out || n_seq < 0 || n_seq > 65535 || heads <= 0 || head_dim <= 0 || max_len <= 0 ||
        row_stride < (long)heads * head_dim || out_row_stride < (long)heads * head_dim || seq_stride < 0 || out_seq_stride < 0)
        return PIMB200_ERR_BAD_ARG;
    const size_t smem = (size_t)max_len * (head_dim + 2) * 2 + (size_t)max_len * head_dim * 2 +
                        (size_t)(kBlockAttnThreads / 32) * (head_dim + max_len) * sizeof(float);
    if (smem > 48 * 1024 || head_dim % 2 != 0) return PIMB200_ERR_UNSUPPORTED;
    attention_block_kernel<<<dim3((unsigned)heads, (unsigned)n_seq), kBlockAttnThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(q), static_cast<const __half*>(k), static_cast<const __half*>(v), lengths,
        static_cast<__half*>(out), max_len, head_dim, row_stride, seq_stride, out_row_stride, out_seq_stride, scale);
    return launch_status();
}

extern "C" int pimb200_topk_rows(const void* x, void* values, long long* idx, long rows, long cols, int k, int largest,
                                 void* stream) {
    if (rows == 0 || k == 0) return PIMB200_OK;
    if (!x || !values || !idx || !rows_ok(rows, cols) || k < 0) return PIMB200_ERR_BAD_ARG;
    if (k > cols) return PIMB200_ERR_BAD_ARG;
    if (k > 64) return PIMB200_ERR_UNSUPPORTED;      // k passes over the row: meant for beam widths, not for sorting
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cols >= kWideRow)
        topk_rows_kernel<1024><<<(unsigned)rows, 1024, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(values), idx,
                                                               cols, k, largest ? 1 : 0);
    else
        topk_rows_kernel<128><<<(unsigned)rows, 128, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(values), idx,
                                                             cols, k, largest ? 1 : 0);
    return launch_status();
}
