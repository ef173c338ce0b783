// Fused multi-layer LSTM forward (inference), fp16 storage / fp32 accumulate.
//
// Math (PyTorch gate order i,f,g,o — the order at::lstm uses, which the reference calls at
// runtime/source/executor/op_executor/aten_ops.cpp:328-344):
//     z      = W_ih x_t + b_ih + W_hh h_{t-1} + b_hh
//     c_t    = sigmoid(z_f) * c_{t-1} + sigmoid(z_i) * tanh(z_g)
//     h_t    = sigmoid(z_o) * tanh(c_t)
//
// Structure per (layer, direction):
//   1. whole-sequence input projection  G[T*B, 4H] = X · Wp_ih^T  (one dense GEMM, fp32 result)
//   2. the recurrence over T:
//        streamed   — one launch per timestep; W_hh is re-read (from L2/HBM) every step with
//                     128-bit loads; any B, any H; the form used by seq_len==1 decoder calls
//        persistent — one cooperative launch for all T steps; every CTA keeps its slice of W_hh on
//                     chip for the whole sequence and the CTAs exchange the new hidden states through
//                     L2 once per step (16-byte records + per-CTA step flags + bulk-copy gather).
//                     Defaults (H <= 1024, slice in registers as mma fragments): 1..32 lock-step
//                     sequences run lstm_persistent_wide_kernel (exchange on the compute warps: the
//                     shortest critical path when there is little to overlap), 33..128 run
//                     lstm_persistent_pipe_kernel (warp-specialised; independent sequence groups,
//                     so one group's exchange runs under the others' arithmetic; 65..128 as two
//                     batch halves on CTAs of 16 units).  Kept beside them: the K-split kernel with
//                     the slice in shared memory (2..32 sequences, any H that fits), the tagged-word
//                     kernel (up to 8 sequences, data and flag in one 16-byte word) and an opt-in
//                     tcgen05 variant (measured slower).
// Weights are stored gate-interleaved (packed row u*4+g = original row g*H+u) so the four gate
// rows of one hidden unit are contiguous and its four pre-activations are one float4 of G.
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "tc_common.cuh"

namespace pimb200 {
int launch_gemm_wx_simt(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                        int ldy, int act, int y_is_f32, cudaStream_t st);
int launch_gemm_wx(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                   int ldy, int act, int y_is_f32, cudaStream_t st);
int launch_gemm_wx_time_major(const __half* W, const __half* X, void* Y, int N, int K, int J, int ldx, int ldy, int batch,
                              cudaStream_t st);
}  // namespace pimb200

using namespace pimb200;

// ---------------------------------------------------------------------------------------------
// weight packing
// ---------------------------------------------------------------------------------------------
__global__ void lstm_pack_matrix_kernel(const __half* __restrict__ src, __half* __restrict__ dst, int H, int cols) {
    // dst[(u*4+g), :] = src[(g*H+u), :]
    const size_t total = (size_t)4 * H * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t prow = i / cols;
        const int c = (int)(i - prow * cols);
        const int u = (int)(prow >> 2), g = (int)(prow & 3);
        dst[i] = src[((size_t)g * H + u) * cols + c];
    }
}
__global__ void lstm_pack_bias_kernel(const __half* __restrict__ b_ih, const __half* __restrict__ b_hh,
                                      float* __restrict__ dst, int H) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 4 * H) return;
    const int u = i >> 2, g = i & 3;
    float v = 0.f;
    if (b_ih) v += __half2float(b_ih[g * H + u]);
    if (b_hh) v += __half2float(b_hh[g * H + u]);
    dst[i] = v;
}

namespace pimb200 {
void lstm_pack_matrix(const __half* src, __half* dst, int H, int cols, cudaStream_t st) {
    lstm_pack_matrix_kernel<<<296, 256, 0, st>>>(src, dst, H, cols);
}
void lstm_pack_bias(const __half* b_ih, const __half* b_hh, float* dst, int H, cudaStream_t st) {
    lstm_pack_bias_kernel<<<ceil_div(4 * H, 256), 256, 0, st>>>(b_ih, b_hh, dst, H);
}
}  // namespace pimb200

// ---------------------------------------------------------------------------------------------
// streamed recurrence: one launch per timestep
// ---------------------------------------------------------------------------------------------
struct StepArgs {
    const __half* Whh;        // packed [4H, H]
    const float* bias;        // packed [4H]
    const float* G;           // gate pre-activations of this timestep, sequence b at G + b*g_bstride
    long g_bstride;
    const __half* hprev_seq;  // h_{t-1} of sequence b at hprev_seq + b*hp_bstride, valid for b < n_prev
    long hp_bstride;
    int n_prev;
    const __half* h0;         // initial state of sequence b at h0 + b*H (NULL = zeros), used for b >= n_prev
    float* c;                 // running cell state, fp32 [B, H]
    __half* hout;             // h_t of sequence b at hout + b*ho_bstride
    long ho_bstride;
    __half* hn;               // optional final-state outputs [B, H]
    __half* cn;
    int H;
    int B;
};

template <int BT, bool VEC>
__global__ void __launch_bounds__(256) lstm_step_kernel(StepArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int u = blockIdx.x * (blockDim.x >> 5) + warp;
    if (u >= a.H) return;
    const int H = a.H;
    const __half* w = a.Whh + (size_t)u * 4 * H;
    for (int b0 = 0; b0 < a.B; b0 += BT) {
        float acc[4][BT];
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int j = 0; j < BT; ++j) acc[g][j] = 0.f;
        const __half* hp[BT];
#pragma unroll
        for (int j = 0; j < BT; ++j) {
            const int b = min(b0 + j, a.B - 1);
            hp[j] = (b < a.n_prev) ? a.hprev_seq + (size_t)b * a.hp_bstride : (a.h0 ? a.h0 + (size_t)b * H : nullptr);
        }
        if (VEC) {
            const int H8 = H >> 3;
#pragma unroll 2
            for (int c = lane; c < H8; c += 32) {
                uint4 wv[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) wv[g] = __ldg(reinterpret_cast<const uint4*>(w + (size_t)g * H) + c);
#pragma unroll
                for (int j = 0; j < BT; ++j) {
                    if (hp[j]) {
                        float xf[8];
                        widen8(__ldcg(reinterpret_cast<const uint4*>(hp[j]) + c), xf);
#pragma unroll
                        for (int g = 0; g < 4; ++g) acc[g][j] = dot8f(wv[g], xf, acc[g][j]);
                    }
                }
            }
        } else {
            for (int k = lane; k < H; k += 32) {
                float wf[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) wf[g] = __half2float(w[(size_t)g * H + k]);
#pragma unroll
                for (int j = 0; j < BT; ++j) {
                    if (hp[j]) {
                        const float hv = __half2float(__ldcg(hp[j] + k));
#pragma unroll
                        for (int g = 0; g < 4; ++g) acc[g][j] = fmaf(wf[g], hv, acc[g][j]);
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int j = 0; j < BT; ++j) acc[g][j] = warp_sum(acc[g][j]);
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < BT; ++j) {
                const int b = b0 + j;
                if (b >= a.B) break;
                const float* gx = a.G + (size_t)b * a.g_bstride + (size_t)u * 4;
                const float zi = acc[0][j] + gx[0] + a.bias[u * 4 + 0];
                const float zf = acc[1][j] + gx[1] + a.bias[u * 4 + 1];
                const float zg = acc[2][j] + gx[2] + a.bias[u * 4 + 2];
                const float zo = acc[3][j] + gx[3] + a.bias[u * 4 + 3];
                float* cp = a.c + (size_t)b * H + u;
                const float cnew = sigmoidf_(zf) * (*cp) + sigmoidf_(zi) * tanhf_(zg);
                const float hnew = sigmoidf_(zo) * tanhf_(cnew);
                *cp = cnew;
                const __half hh = __float2half_rn(hnew);
                a.hout[(size_t)b * a.ho_bstride + u] = hh;
                if (a.hn) a.hn[(size_t)b * H + u] = hh;
                if (a.cn) a.cn[(size_t)b * H + u] = __float2half_rn(cnew);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// decode form (seq_len == 1): one launch per layer and direction computes the whole cell,
//     z = W_ih x + W_hh h0 + b,  c = sigma(z_f) c0 + sigma(z_i) tanh(z_g),  h = sigma(z_o) tanh(c),
// a warp per hidden unit streaming its four rows of both matrices once (128-bit loads that bypass L1), x and h0
// through L1.  Replaces the projection GEMM + state initialisation + step kernel of the general path, which cost
// three launches per layer where an autoregressive decoder calls aten::lstm once per token.
// ---------------------------------------------------------------------------------------------
struct CellArgs {
    const __half* Wih;   // packed [4H, I]
    const __half* Whh;   // packed [4H, H]
    const float* bias;   // packed [4H]
    const __half* x;     // input of sequence b at x + b*x_bstride
    long x_bstride;
    const __half* h0;    // [B, H] or NULL
    const __half* c0;    // [B, H] or NULL
    __half* y;           // h of sequence b at y + b*y_bstride
    long y_bstride;
    __half* hn;          // optional [B, H]
    __half* cn;          // optional [B, H]
    int I, H, B;
};

template <int BT>
__global__ void __launch_bounds__(256) lstm_cell_kernel(CellArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int u = blockIdx.x * (blockDim.x >> 5) + warp;
    if (u >= a.H) return;
    const int H = a.H, I = a.I;
    const __half* wi = a.Wih + (size_t)u * 4 * I;
    const __half* wh = a.Whh + (size_t)u * 4 * H;
    for (int b0 = 0; b0 < a.B; b0 += BT) {
        float acc[4][BT];
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int j = 0; j < BT; ++j) acc[g][j] = 0.f;
        const int I8 = I >> 3, H8 = H >> 3;
#pragma unroll 2
        for (int c = lane; c < I8; c += 32) {
            uint4 wv[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) wv[g] = ldg_stream_v4(reinterpret_cast<const uint4*>(wi + (size_t)g * I) + c);
#pragma unroll
            for (int j = 0; j < BT; ++j) {
                const int b = min(b0 + j, a.B - 1);
                float xf[8];
                widen8(__ldg(reinterpret_cast<const uint4*>(a.x + (size_t)b * a.x_bstride) + c), xf);
#pragma unroll
                for (int g = 0; g < 4; ++g) acc[g][j] = dot8f(wv[g], xf, acc[g][j]);
            }
        }
        if (a.h0) {
#pragma unroll 2
            for (int c = lane; c < H8; c += 32) {
                uint4 wv[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) wv[g] = ldg_stream_v4(reinterpret_cast<const uint4*>(wh + (size_t)g * H) + c);
#pragma unroll
                for (int j = 0; j < BT; ++j) {
                    const int b = min(b0 + j, a.B - 1);
                    float xf[8];
                    widen8(__ldg(reinterpret_cast<const uint4*>(a.h0 + (size_t)b * H) + c), xf);
#pragma unroll
                    for (int g = 0; g < 4; ++g) acc[g][j] = dot8f(wv[g], xf, acc[g][j]);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int j = 0; j < BT; ++j) acc[g][j] = warp_sum(acc[g][j]);
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < BT; ++j) {
                const int b = b0 + j;
                if (b >= a.B) break;
                const float zi = acc[0][j] + a.bias[u * 4 + 0], zf = acc[1][j] + a.bias[u * 4 + 1],
                            zg = acc[2][j] + a.bias[u * 4 + 2], zo = acc[3][j] + a.bias[u * 4 + 3];
                const float cprev = a.c0 ? __half2float(a.c0[(size_t)b * H + u]) : 0.f;
                const float cnew = sigmoidf_(zf) * cprev + sigmoidf_(zi) * tanhf_(zg);
                const __half hh = __float2half_rn(sigmoidf_(zo) * tanhf_(cnew));
                a.y[(size_t)b * a.y_bstride + u] = hh;
                if (a.hn) a.hn[(size_t)b * H + u] = hh;
                if (a.cn) a.cn[(size_t)b * H + u] = __float2half_rn(cnew);
            }
        }
    }
}

// Decode form for 8 or more sequences in lock step (a batched decode step: one token for each of B sentences): the
// cell kernel above would stream both matrices once per four sequences, so the two products run as GEMMs over the B
// rows (one pass over each matrix whatever B is) into fp32 gate terms, and this kernel applies bias and gate math:
// a thread per (sequence, hidden unit), the unit's four gate terms one 16-byte load from each product.
constexpr int kCellGemmMinB = 8;
struct CellPointArgs {
    const float* Gx;     // [B, 4H]  W_ih x, packed gate order (unit-major)
    const float* Gh;     // [B, 4H]  W_hh h0, or NULL when h0 is zero
    const float* bias;   // packed [4H]
    const __half* c0;    // [B, H] or NULL
    __half* y;           // h of sequence b at y + b*y_bstride
    long y_bstride;
    __half* hn;          // optional [B, H]
    __half* cn;          // optional [B, H]
    int H, B;
    const __half* res;   // optional residual rows: y = h + res (fp16 add of the rounded h, as a separate add would do)
    long res_bstride;
};

__global__ void __launch_bounds__(256) lstm_cell_point_kernel(CellPointArgs a) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)a.B * a.H) return;
    const int b = (int)(idx / a.H), u = (int)(idx % a.H);
    float4 z = *reinterpret_cast<const float4*>(a.Gx + ((size_t)b * a.H + u) * 4);
    if (a.Gh) {
        const float4 zh = *reinterpret_cast<const float4*>(a.Gh + ((size_t)b * a.H + u) * 4);
        z.x += zh.x; z.y += zh.y; z.z += zh.z; z.w += zh.w;
    }
    const float4 bb = *reinterpret_cast<const float4*>(a.bias + (size_t)u * 4);
    const float cprev = a.c0 ? __half2float(a.c0[(size_t)b * a.H + u]) : 0.f;
    const float cnew = sigmoidf_(z.y + bb.y) * cprev + sigmoidf_(z.x + bb.x) * tanhf_(z.z + bb.z);
    const __half hh = __float2half_rn(sigmoidf_(z.w + bb.w) * tanhf_(cnew));
    a.y[(size_t)b * a.y_bstride + u] =
        a.res ? __float2half_rn(__half2float(hh) + __half2float(a.res[(size_t)b * a.res_bstride + u])) : hh;
    if (a.hn) a.hn[(size_t)b * a.H + u] = hh;
    if (a.cn) a.cn[(size_t)b * a.H + u] = __float2half_rn(cnew);
}

__global__ void lstm_init_c_kernel(float* __restrict__ c, const __half* __restrict__ c0, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) c[i] = c0 ? __half2float(c0[i]) : 0.f;
}
// final states of sequences that never became active cannot occur (batch_sizes[0] == B), but the
// padded path with T steps needs hn/cn even when the caller passes h0 only: handled by the step kernel.

// ---------------------------------------------------------------------------------------------
// persistent weight-stationary recurrence (1 <= B <= 8 sequences in lock step)
//
// Grid: one CTA per SM (cooperative launch, so all CTAs are co-resident).  CTA c owns U = ceil(H/#SM) <= 7
// hidden units = 4U gate rows of W_hh, kept in shared memory for all T steps (rows padded to 32 = two
// m16 tiles; row pitch H+8 halves so ldmatrix is bank-conflict free).
// Per step:
//   1. Z[32 x 8] = W_slice[32 x H] . Hprev[H x 8]  on the tensor cores (mma.sync m16n8k16, fp32
//      accumulate): column n of the B operand is the hidden state of sequence n, so up to eight
//      sequences cost the same tensor work as one.  The 8 warps split K; partial sums meet in shared
//      memory.
//   2. thread (row, n) finishes one sum; warp j then holds the four gates of unit j for all sequences,
//      lanes 0..B-1 add the hoisted input projection and bias, run the gate math and keep c in fp32
//      registers for the whole sequence.
//   3. the CTA publishes, per sequence, ONE 16-byte word {7 x fp16 hidden values, 16-bit step tag} with a
//      single-copy-atomic st.relaxed.gpu.b128 into every replica of the exchange buffer.
//   4. the threads poll the B * n_cta words of this CTA's replica until each carries the current step's
//      tag (data and flag arrive together: one L2 round trip, no separate barrier) and scatter the values
//      into the next step's h vectors in shared memory.
// Every wait is bounded: after poll_limit polls the CTA records PIMB200_ERR_TIMEOUT in the status word
// and leaves; the others see the status (or run out themselves) and leave too.
// ---------------------------------------------------------------------------------------------
constexpr int kPersistPollLimit = 1 << 21;  // bounded wait: ~seconds, then the kernel gives up
constexpr int kXchgCopies = 16;             // replicas of the hidden-state exchange buffer
constexpr int kXchgWords = 160;             // 16-byte words per replica, parity and sequence (>= CTAs in the grid)
constexpr int kPersistThreads = 256;
constexpr int kPersistWarps = kPersistThreads / 32;
constexpr int kPersistRows = 32;            // padded gate rows per CTA
constexpr int kUnitsPerWord = 7;
constexpr int kPersistMaxB = 8;             // sequences per launch = columns of one mma tile
constexpr int kPollItems = kPersistMaxB * kXchgWords / kPersistThreads;  // words a thread may have to gather
constexpr int kXchgMaxStride = 8;           // largest spacing of exchange words, in 16-byte units (8 = one word per 128-byte line)
constexpr size_t kXchgBytes = (size_t)kXchgCopies * 2 * kPersistMaxB * kXchgWords * 16 * kXchgMaxStride;

struct PersistArgs {
    const __half* Whh;      // packed [4H, H]
    const float* bias;      // packed [4H]
    const float* G;         // gate pre-activations of (t, n) at G + t*g_tstride + n*g_bstride (floats)
    long g_tstride, g_bstride;
    const __half* h0;       // [B][H] or NULL
    const __half* c0;       // [B][H] or NULL
    __half* y;              // h_t of sequence n at y + t*y_tstride + n*y_bstride + u
    long y_tstride, y_bstride;
    __half* hn;             // optional [B][H]
    __half* cn;             // optional [B][H]
    uint4* xchg;            // [copies][2][kPersistMaxB][kXchgWords] exchange words
    int copies;
    int wstride;            // spacing of consecutive exchange words in 16-byte units
    uint32_t tag_base;      // tag of step s output = (tag_base + s + 1) & 0xffff
    int* status;            // device status block: [0] sticky error code, [1] generation of the launch that gave up
    int gen;                // this launch's generation (never 0)
    int H, T, U, B;         // U = hidden units per CTA
    int reverse;
    int poll_limit;
    long long* trace;       // optional diagnostics, 8 int64 per CTA and step: clocks at step start, after publish,
                            // after gather, polls, after mma, after barrier, after gates
};

__device__ __forceinline__ void st_b128_relaxed(uint4* p, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    const unsigned long long lo = ((unsigned long long)y << 32) | x, hi = ((unsigned long long)w << 32) | z;
    asm volatile("{ .reg .b128 q; mov.b128 q, {%1, %2}; st.relaxed.gpu.global.b128 [%0], q; }" ::"l"(p), "l"(lo), "l"(hi)
                 : "memory");
}
__device__ __forceinline__ void ld_b128_relaxed(const uint4* p, uint32_t& x, uint32_t& y, uint32_t& z, uint32_t& w) {
    unsigned long long lo, hi;
    asm volatile("{ .reg .b128 q; ld.relaxed.gpu.global.b128 q, [%2]; mov.b128 {%0, %1}, q; }"
                 : "=l"(lo), "=l"(hi)
                 : "l"(p)
                 : "memory");
    x = (uint32_t)lo; y = (uint32_t)(lo >> 32); z = (uint32_t)hi; w = (uint32_t)(hi >> 32);
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kPersistThreads, 1) lstm_persistent_kernel(PersistArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, U = a.U, T = a.T, B = a.B;
    const int pitch = H + 8;                                               // halves per padded row (weights and h)
    __half* Ws = reinterpret_cast<__half*>(smem_raw);                      // [32][pitch]
    __half* hs = Ws + (size_t)kPersistRows * pitch;                        // [2][B][pitch]
    float* part = reinterpret_cast<float*>(hs + (size_t)2 * B * pitch);    // [8 warps][32 rows][8 cols]
    unsigned short* hpub = reinterpret_cast<unsigned short*>(part + kPersistWarps * kPersistRows * 8);  // [8][8]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_cta = gridDim.x;
    const int u0 = blockIdx.x * U;
    const int nu = min(U, H - u0);  // units this CTA owns
    const int ktiles = H >> 4;
    const int ws = a.wstride;
    const uint4* my_copy = a.xchg + (size_t)(blockIdx.x % a.copies) * 2 * kPersistMaxB * kXchgWords * ws;

    // one-time: this CTA's slice of W_hh goes to shared memory and stays there for all T steps
    {
        const int H8 = H >> 3;
        const uint4* src = reinterpret_cast<const uint4*>(a.Whh + (size_t)u0 * 4 * H);
        for (int i = tid; i < kPersistRows * H8; i += kPersistThreads) {
            const int r = i / H8, c8 = i - r * H8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < 4 * nu) v = ldg_stream_v4(src + (size_t)r * H8 + c8);
            *reinterpret_cast<uint4*>(Ws + (size_t)r * pitch + c8 * 8) = v;
        }
    }
    for (int i = tid; i < B * H; i += kPersistThreads) {
        const int n = i / H, k = i - n * H;
        hs[(size_t)n * pitch + k] = a.h0 ? a.h0[i] : __float2half_rn(0.f);
    }
    if (tid < 64) hpub[tid] = 0;

    // gate lanes: warp j owns unit u0+j, its lane n (< B) owns sequence n
    const bool gate_lane = (warp < nu) && (lane < B);
    const int u = u0 + warp;
    float c = 0.f;
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 gx = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gate_lane) {
        c = a.c0 ? __half2float(a.c0[(size_t)lane * H + u]) : 0.f;
        bias4 = *reinterpret_cast<const float4*>(a.bias + (size_t)u * 4);
        const int t0 = a.reverse ? T - 1 : 0;
        gx = __ldcg(reinterpret_cast<const float4*>(a.G + (size_t)t0 * a.g_tstride + (size_t)lane * a.g_bstride +
                                                    (size_t)u * 4));
    }
    // ldmatrix source row/column of this lane inside a 16x16 A tile; B-operand column (sequence) of this lane
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int a_col = (lane >> 4) * 8;
    const int b_n = lane >> 2, b_k = (lane & 3) * 2;
    __syncthreads();

    for (int s = 0; s < T; ++s) {
        const int t = a.reverse ? T - 1 - s : s;
        const __half* hcur = hs + (size_t)(s & 1) * B * pitch;
        long long* tr = a.trace ? a.trace + ((size_t)blockIdx.x * T + s) * 8 : nullptr;
        if (tr && tid == 0) tr[0] = clock64();
        // ---- 1. partial products on the tensor cores; warps split K
        float acc[2][4];
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;
        // four k-tiles per trip: their shared-memory loads are all issued before the first mma
        for (int kt0 = warp; kt0 < ktiles; kt0 += 4 * kPersistWarps) {
            uint32_t b0[4], b1[4], af[4][2][4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int kt = kt0 + q * kPersistWarps;
                const int k0 = min(kt, ktiles - 1) << 4;
                b0[q] = 0u;
                b1[q] = 0u;
                if (b_n < B && kt < ktiles) {  // column n of the B operand = h of sequence n
                    const __half* hp = hcur + (size_t)b_n * pitch + k0 + b_k;
                    b0[q] = *reinterpret_cast<const uint32_t*>(hp);
                    b1[q] = *reinterpret_cast<const uint32_t*>(hp + 8);
                }
#pragma unroll
                for (int m = 0; m < 2; ++m) ldmatrix_x4(af[q][m], Ws + (size_t)(m * 16 + a_row) * pitch + k0 + a_col);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int m = 0; m < 2; ++m) mma_16816(acc[m], af[q][m], b0[q], b1[q]);  // B is zero past the last tile
        }
        if (tr && tid == 0) tr[4] = clock64();
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float* p = part + ((size_t)warp * kPersistRows + m * 16 + (lane >> 2)) * 8 + b_k;
            *reinterpret_cast<float2*>(p) = make_float2(acc[m][0], acc[m][1]);
            *reinterpret_cast<float2*>(p + 8 * 8) = make_float2(acc[m][2], acc[m][3]);
        }
        __syncthreads();
        if (tr && tid == 0) tr[5] = clock64();
        // ---- 2. thread (row = tid/8, n = tid%8) finishes one sum; warp j then holds unit j: lane = gate*8 + n
        {
            float z = 0.f;
#pragma unroll
            for (int w = 0; w < kPersistWarps; ++w) z += part[(size_t)w * kPersistRows * 8 + tid];
            const float zf_ = __shfl_down_sync(0xffffffffu, z, 8);
            const float zg_ = __shfl_down_sync(0xffffffffu, z, 16);
            const float zo_ = __shfl_down_sync(0xffffffffu, z, 24);
            if (gate_lane) {
                const float zi = z + gx.x + bias4.x, zf = zf_ + gx.y + bias4.y, zg = zg_ + gx.z + bias4.z,
                            zo = zo_ + gx.w + bias4.w;
                c = sigmoidf_(zf) * c + sigmoidf_(zi) * tanhf_(zg);
                const __half hh = __float2half_rn(sigmoidf_(zo) * tanhf_(c));
                hpub[lane * 8 + warp] = __half_as_ushort(hh);
                a.y[(size_t)t * a.y_tstride + (size_t)lane * a.y_bstride + u] = hh;
                if (s == T - 1) {
                    if (a.hn) a.hn[(size_t)lane * H + u] = hh;
                    if (a.cn) a.cn[(size_t)lane * H + u] = __float2half_rn(c);
                }
                if (s + 1 < T) {
                    const int tn = a.reverse ? t - 1 : t + 1;
                    gx = __ldcg(reinterpret_cast<const float4*>(a.G + (size_t)tn * a.g_tstride +
                                                                (size_t)lane * a.g_bstride + (size_t)u * 4));
                }
            }
        }
        if (tr && tid == 0) tr[6] = clock64();
        int timed_out = 0, polls = 0;
        if (s + 1 < T) {
            __syncthreads();
            // ---- 3. publish: thread (n, copy) writes sequence n's word into one replica
            const uint32_t tag16 = (a.tag_base + (uint32_t)s + 1u) & 0xffffu;
            if (tid < B * a.copies) {
                const int n = tid / a.copies, cp = tid - n * a.copies;
                const uint4 v = *reinterpret_cast<const uint4*>(hpub + n * 8);
                st_b128_relaxed(a.xchg + ((((size_t)cp * 2 + (s & 1)) * kPersistMaxB + n) * kXchgWords + blockIdx.x) * ws, v.x,
                                v.y, v.z, (v.w & 0xffffu) | (tag16 << 16));
            }
            if (tr && tid == 0) tr[1] = clock64();
            // ---- 4. gather h_s of every sequence from every CTA
            const uint4* src = my_copy + (size_t)(s & 1) * kPersistMaxB * kXchgWords * ws;
            __half* hnext = hs + (size_t)((s + 1) & 1) * B * pitch;
            const int n_items = B * n_cta;
            uint32_t vx[kPollItems], vy[kPollItems], vz[kPollItems], vw[kPollItems];
            unsigned pending = 0u;
#pragma unroll
            for (int k = 0; k < kPollItems; ++k)
                if (tid + k * kPersistThreads < n_items) pending |= 1u << k;
            while (pending) {
#pragma unroll
                for (int k = 0; k < kPollItems; ++k) {
                    if (pending & (1u << k)) {
                        const int item = tid + k * kPersistThreads;
                        const int n = item / n_cta, cta = item - n * n_cta;
                        ld_b128_relaxed(src + ((size_t)n * kXchgWords + cta) * ws, vx[k], vy[k], vz[k], vw[k]);
                    }
                }
#pragma unroll
                for (int k = 0; k < kPollItems; ++k)
                    if ((pending & (1u << k)) && (vw[k] >> 16) == tag16) pending &= ~(1u << k);
                if (!pending) break;
                if (++polls >= a.poll_limit) {
                    timed_out = 1;
                    break;
                }
                if ((polls & 1023) == 0 && status_aborted(a.status, a.gen)) {
                    timed_out = 1;  // another CTA already gave up
                    break;
                }
            }
            if (!timed_out) {
#pragma unroll
                for (int k = 0; k < kPollItems; ++k) {
                    const int item = tid + k * kPersistThreads;
                    if (item < n_items) {
                        const int n = item / n_cta, cta = item - n * n_cta;
                        __half* dst = hnext + (size_t)n * pitch + (size_t)cta * U;
                        const int cnt = min(U, H - cta * U);
                        const uint32_t vals[4] = {vx[k], vy[k], vz[k], vw[k]};
#pragma unroll
                        for (int j = 0; j < kUnitsPerWord; ++j)
                            if (j < cnt) dst[j] = __ushort_as_half((unsigned short)((vals[j >> 1] >> ((j & 1) * 16)) & 0xffffu));
                    }
                }
            } else {
                status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
            }
        }
        if (tr && tid == 0) { tr[2] = clock64(); tr[3] = polls; }
        if (__syncthreads_or(timed_out)) return;  // whole CTA leaves together
    }
}

// ---------------------------------------------------------------------------------------------
// persistent weight-stationary recurrence, batched variant (2 <= B <= 32 sequences in lock step)
//
// Same ownership and tensor-core matvec as above (8 hidden units = 32 gate rows per CTA, H/8 CTAs), with NT tiles of
// 8 sequences per mma pass, but a different exchange: strong (relaxed.gpu) loads cost the SM a few cycles each, so
// polling B * n_cta tagged words does not scale with B.  Here a CTA writes its B x 8 new hidden values with plain
// 16-byte stores, fences, and raises ONE 32-bit step flag; readers poll the n_cta flags (strong loads), fence, and
// then fetch the data with ordinary coalesced 16-byte loads.  Two L2 round trips per step instead of one, but the
// volume moves at full L2 bandwidth.
// ---------------------------------------------------------------------------------------------
constexpr int kBulkMaxB = 64;              // sequences per launch of the batched variants
constexpr int kBulkFlagCopies = 8;         // replicas of the step flags

struct BulkArgs {
    const __half* Whh;
    const float* bias;
    const float* G;
    long g_tstride, g_bstride;
    const __half* h0;
    const __half* c0;
    __half* y;
    long y_tstride, y_bstride;
    int y_vec;              // 1 = (t, n) rows of y are 16-byte aligned: one uint4 store per sequence
    __half* hn;
    __half* cn;
    uint4* data;            // [2 parities][n_cta][BP] 16-byte records: the 8 hidden values of (cta, sequence)
    uint32_t* flags;        // [kBulkFlagCopies][2 parities][n_cta] step tags, one per 128-byte line
    uint32_t tag_base;      // flag value of step s = tag_base + s + 1
    int* status;            // as in PersistArgs
    int gen;
    int H, T, B;
    int reverse;
    int poll_limit;
    long long* trace;       // optional diagnostics, 8 clocks per CTA and step
};

template <int NT>
__global__ void __launch_bounds__(kPersistThreads, 1) lstm_persistent_bulk_kernel(BulkArgs a) {
    constexpr int BP = NT * 8;  // sequences, padded to whole mma tiles
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, T = a.T, B = a.B;
    const int pitch = H + 8;
    __half* Ws = reinterpret_cast<__half*>(smem_raw);                         // [32][pitch]
    __half* hs = Ws + (size_t)kPersistRows * pitch;                           // [BP][pitch]
    float* part = reinterpret_cast<float*>(hs + (size_t)BP * pitch);          // [8 warps][32 rows][BP]
    unsigned short* hpub = reinterpret_cast<unsigned short*>(part + (size_t)kPersistWarps * kPersistRows * BP);  // [BP][8]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_cta = gridDim.x, cta = blockIdx.x;
    const int u0 = cta * 8;
    const int ktiles = H >> 4;
    {
        const int H8 = H >> 3;
        const uint4* src = reinterpret_cast<const uint4*>(a.Whh + (size_t)u0 * 4 * H);
        for (int i = tid; i < kPersistRows * H8; i += kPersistThreads) {
            const int r = i / H8, c8 = i - r * H8;
            *reinterpret_cast<uint4*>(Ws + (size_t)r * pitch + c8 * 8) = ldg_stream_v4(src + (size_t)r * H8 + c8);
        }
    }
    for (int i = tid; i < BP * H; i += kPersistThreads) {
        const int n = i / H, k = i - n * H;
        hs[(size_t)n * pitch + k] = (n < B && a.h0) ? a.h0[(size_t)n * H + k] : __float2half_rn(0.f);
    }
    for (int i = tid; i < BP * 8; i += kPersistThreads) hpub[i] = 0;

    // gate thread (unit = warp, sequence = lane)
    const bool gate_thread = lane < B;
    const int u = u0 + warp;
    float c = 0.f;
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f), gx = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gate_thread) {
        c = a.c0 ? __half2float(a.c0[(size_t)lane * H + u]) : 0.f;
        bias4 = *reinterpret_cast<const float4*>(a.bias + (size_t)u * 4);
        const int t0 = a.reverse ? T - 1 : 0;
        gx = __ldcg(reinterpret_cast<const float4*>(a.G + (size_t)t0 * a.g_tstride + (size_t)lane * a.g_bstride +
                                                    (size_t)u * 4));
    }
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int a_col = (lane >> 4) * 8;
    const int b_n = lane >> 2, b_k = (lane & 3) * 2;
    __syncthreads();

    for (int s = 0; s < T; ++s) {
        const int t = a.reverse ? T - 1 - s : s;
        const int par = s & 1;
        long long* tr = a.trace ? a.trace + ((size_t)blockIdx.x * T + s) * 8 : nullptr;
        if (tr && tid == 0) tr[0] = clock64();
        // ---- 1. Z[32 x BP] partial products, warps split K
        float acc[2][NT][4];
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[m][nt][i] = 0.f;
        for (int kt0 = warp; kt0 < ktiles; kt0 += 2 * kPersistWarps) {
            uint32_t af[2][2][4], b0[2][NT], b1[2][NT];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int kt = kt0 + q * kPersistWarps;
                const bool live = kt < ktiles;
                const int k0 = min(kt, ktiles - 1) << 4;
#pragma unroll
                for (int m = 0; m < 2; ++m) ldmatrix_x4(af[q][m], Ws + (size_t)(m * 16 + a_row) * pitch + k0 + a_col);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const __half* hp = hs + (size_t)(nt * 8 + b_n) * pitch + k0 + b_k;
                    b0[q][nt] = live ? *reinterpret_cast<const uint32_t*>(hp) : 0u;
                    b1[q][nt] = live ? *reinterpret_cast<const uint32_t*>(hp + 8) : 0u;
                }
            }
#pragma unroll
            for (int q = 0; q < 2; ++q)
#pragma unroll
                for (int m = 0; m < 2; ++m)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) mma_16816(acc[m][nt], af[q][m], b0[q][nt], b1[q][nt]);
        }
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float* p = part + ((size_t)warp * kPersistRows + m * 16 + (lane >> 2)) * BP + nt * 8 + b_k;
                *reinterpret_cast<float2*>(p) = make_float2(acc[m][nt][0], acc[m][nt][1]);
                *reinterpret_cast<float2*>(p + 8 * BP) = make_float2(acc[m][nt][2], acc[m][nt][3]);
            }
        __syncthreads();
        if (tr && tid == 0) tr[1] = clock64();
        // ---- 2. gates of (unit = warp, sequence = lane)
        if (gate_thread) {
            float z[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int w = 0; w < kPersistWarps; ++w)
#pragma unroll
                for (int g = 0; g < 4; ++g) z[g] += part[((size_t)w * kPersistRows + warp * 4 + g) * BP + lane];
            const float zi = z[0] + gx.x + bias4.x, zf = z[1] + gx.y + bias4.y, zg = z[2] + gx.z + bias4.z,
                        zo = z[3] + gx.w + bias4.w;
            c = sigmoidf_(zf) * c + sigmoidf_(zi) * tanhf_(zg);
            const __half hh = __float2half_rn(sigmoidf_(zo) * tanhf_(c));
            hpub[lane * 8 + warp] = __half_as_ushort(hh);
            if (!a.y_vec) a.y[(size_t)t * a.y_tstride + (size_t)lane * a.y_bstride + u] = hh;
            if (s == T - 1) {
                if (a.hn) a.hn[(size_t)lane * H + u] = hh;
                if (a.cn) a.cn[(size_t)lane * H + u] = __float2half_rn(c);
            }
            if (s + 1 < T) {
                const int tn = a.reverse ? t - 1 : t + 1;
                gx = __ldcg(reinterpret_cast<const float4*>(a.G + (size_t)tn * a.g_tstride + (size_t)lane * a.g_bstride +
                                                            (size_t)u * 4));
            }
        }
        __syncthreads();
        if (tr && tid == 0) tr[2] = clock64();
        // ---- 3. publish: one 16-byte record per sequence, to the output tensor and to the exchange buffer
        if (tid < B) {
            const uint4 v = *reinterpret_cast<const uint4*>(hpub + tid * 8);
            if (a.y_vec) *reinterpret_cast<uint4*>(a.y + (size_t)t * a.y_tstride + (size_t)tid * a.y_bstride + u0) = v;
            if (s + 1 < T) {
                a.data[((size_t)par * n_cta + cta) * BP + tid] = v;
                __threadfence();  // the record is visible device-wide before the flag can be
            }
        }
        if (s + 1 == T) break;
        __syncthreads();
        if (tr && tid == 0) tr[3] = clock64();
        const uint32_t tag = a.tag_base + (uint32_t)s + 1u;
        // the flag goes to every replica; each flag has a 128-byte line of its own, so a line is polled by n_cta/replicas CTAs
        if (tid < kBulkFlagCopies)
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(a.flags + (((size_t)tid * 2 + par) * n_cta + cta) * 32), "r"(tag) : "memory");
        // ---- 4. wait for every CTA's flag of this step
        int timed_out = 0;
        if (tid < n_cta) {
            const uint32_t* f = a.flags + (((size_t)(cta % kBulkFlagCopies) * 2 + par) * n_cta + tid) * 32;
            int polls = 0;
            while (true) {
                uint32_t v;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                if (v == tag) break;
                if (++polls >= a.poll_limit) { timed_out = 1; break; }
                if ((polls & 1023) == 0 && status_aborted(a.status, a.gen)) { timed_out = 1; break; }
            }
            if (timed_out) status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
            if (tr && tid == 0) tr[4] = clock64();
            __threadfence();  // acquire side: loads below are ordered after the flag reads
            if (tr && tid == 0) tr[5] = clock64();
        }
        if (__syncthreads_or(timed_out)) return;
        if (tr && tid == 0) tr[6] = clock64();
        // ---- 5. fetch all records with plain coalesced loads: item = (cta, sequence)
        {
            const uint4* src = a.data + (size_t)par * n_cta * BP;
            const int items = n_cta * BP;
            for (int i = tid; i < items; i += kPersistThreads) {
                const int n = i % BP, j = i / BP;
                if (n < B) *reinterpret_cast<uint4*>(hs + (size_t)n * pitch + j * 8) = src[i];
            }
        }
        __syncthreads();
        if (tr && tid == 0) tr[7] = clock64();
    }
}

// ---------------------------------------------------------------------------------------------
// wide variant of the batched persistent recurrence (up to 64 sequences, H a multiple of 16 up to 1024): the same
// exchange protocol, but the CTA's slice of W_hh lives in REGISTERS as mma A fragments for the whole launch.  Warp w
// owns k-tiles kq, kq+4, kq+8, ... (kq = w & 3) of both 16-row m-tiles and one half of the sequence tiles
// (nh = w >> 2), so per k-tile it reads only B fragments from shared memory (1 KiB for 8 mma.sync; with A staged in
// shared memory the tensor-core phase was bound by shared-memory bandwidth, 512 KiB per step).  The four K-partials
// of a tile meet in a padded fp32 buffer (the four gates of a unit side by side, so a gate thread fetches a partial
// with one 128-bit load) that the gate threads sum.
// The gather of the exchanged hidden states is one contiguous block, fetched by the bulk-copy engine: each warp
// polls the flags of one group of CTAs and issues the copy of that group's records, all completing on one mbarrier.
// ---------------------------------------------------------------------------------------------
constexpr int kWideThreads = kPersistThreads;
constexpr int kWideKq = 4;         // K-split of the tensor-core phase across warps
constexpr int kWideMaxKtw = 16;    // k-tiles per warp held in registers (H <= 1024)

template <int NT>  // 2, 4 or 8 tiles of 8 sequences
__global__ void __launch_bounds__(kWideThreads, 1) lstm_persistent_wide_kernel(BulkArgs a) {
    constexpr int BP = NT * 8;
    constexpr int NH = NT / 2;                       // n-tiles per warp
    constexpr int ZP = BP + 1;                       // padded sequence pitch of the partial sums: [kq][unit][ZP][gate]
    constexpr int PPT = (8 * BP + kPersistThreads - 1) / kPersistThreads;  // (unit, sequence) pairs per gate thread: 1 or 2
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, T = a.T, B = a.B;
    // hidden states in the layout of the exchange records: hs[j][n][8] = units 8j..8j+7 of sequence n.  The gather is
    // then one contiguous copy, and an mma B fragment (k = 16kt + 2t (+8), column n) reads 128 contiguous bytes per
    // warp: no padding, no bank conflicts.
    __half* hs = reinterpret_cast<__half*>(smem_raw);                         // [H/8][BP][8]
    float* zpart = reinterpret_cast<float*>(hs + (size_t)BP * H);             // [kWideKq][8 units][ZP][4 gates]
    unsigned short* hpub = reinterpret_cast<unsigned short*>(zpart + (size_t)kWideKq * 8 * ZP * 4);  // [BP][8]
    uint64_t* gbar = reinterpret_cast<uint64_t*>(hpub + (size_t)BP * 8);
    const uint32_t gbar_addr = (uint32_t)__cvta_generic_to_shared(gbar);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_cta = gridDim.x, cta = blockIdx.x;
    const int u0 = cta * 8;
    const int ktiles = H >> 4;
    const int cpw = (n_cta + kPersistWarps - 1) / kPersistWarps;   // CTAs whose flags and records one warp handles
    if (tid == 0) {
        pimb200::tc::mbar_init(gbar_addr, (uint32_t)((n_cta + cpw - 1) / cpw));   // one arrival per issuing warp
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int kq = warp & (kWideKq - 1), nh = (warp >> 2) & 1;
    const int b_n = lane >> 2, b_k = (lane & 3) * 2;
    // A fragments of this warp: afrag[i][m] = rows 16m..16m+15 of the slice, k-tile kWideKq*i + kq
    uint32_t afrag[kWideMaxKtw][2][4];
    {
        const __half* wbase = a.Whh + (size_t)u0 * 4 * H;
#pragma unroll
        for (int i = 0; i < kWideMaxKtw; ++i) {
#pragma unroll
            for (int m = 0; m < 2; ++m) {
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    afrag[i][m][r] = 0u;
                    if (kWideKq * i + kq < ktiles) {
                        const int row = m * 16 + b_n + (r & 1) * 8;
                        const int k = (kWideKq * i + kq) * 16 + b_k + (r >> 1) * 8;
                        afrag[i][m][r] = __ldg(reinterpret_cast<const uint32_t*>(wbase + (size_t)row * H + k));
                    }
                }
            }
        }
    }
    for (int i = tid; i < BP * H; i += kWideThreads) {
        const int n = i / H, k = i - n * H;
        hs[((size_t)(k >> 3) * BP + n) * 8 + (k & 7)] = (n < B && a.h0) ? a.h0[(size_t)n * H + k] : __float2half_rn(0.f);
    }
    for (int i = tid; i < BP * 8; i += kWideThreads) hpub[i] = 0;

    // gate pairs of this thread: pair p = tid + q*256 -> unit p / BP, sequence p % BP
    int gu[PPT], gn[PPT];
    bool live[PPT];
    float c[PPT];
    float4 bias4[PPT], gx[PPT];
#pragma unroll
    for (int q = 0; q < PPT; ++q) {
        const int p_ = tid + q * kPersistThreads;
        gu[q] = p_ / BP;
        gn[q] = p_ - gu[q] * BP;
        live[q] = p_ < 8 * BP && gn[q] < B;
        if (p_ >= 8 * BP) gu[q] = gn[q] = 0;   // threads beyond the pairs (16 sequences) idle through the gate phase
        c[q] = 0.f;
        bias4[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        gx[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live[q]) {
            const int u = u0 + gu[q];
            c[q] = a.c0 ? __half2float(a.c0[(size_t)gn[q] * H + u]) : 0.f;
            bias4[q] = *reinterpret_cast<const float4*>(a.bias + (size_t)u * 4);
            const int t0 = a.reverse ? T - 1 : 0;
            gx[q] = __ldcg(reinterpret_cast<const float4*>(a.G + (size_t)t0 * a.g_tstride + (size_t)gn[q] * a.g_bstride +
                                                           (size_t)u * 4));
        }
    }
    __syncthreads();

    for (int s = 0; s < T; ++s) {
        const int t = a.reverse ? T - 1 - s : s;
        const int par = s & 1;
        long long* tr = a.trace ? a.trace + ((size_t)blockIdx.x * T + s) * 8 : nullptr;
        if (tr && tid == 0) tr[0] = clock64();
        // ---- 1. K-partial Z tiles of this warp
        {
            float acc[2][NH][4];
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int j = 0; j < NH; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[m][j][i] = 0.f;
            const __half* brow = hs + ((size_t)(nh * NH * 8 + b_n)) * 8 + b_k;   // + (2kt [+1]) * BP * 8 per k-tile
#pragma unroll
            for (int i = 0; i < kWideMaxKtw; ++i) {
                if (kWideKq * i + kq < ktiles) {   // warp-uniform
                    const int kt = kWideKq * i + kq;
                    const __half* hp = brow + (size_t)(2 * kt) * BP * 8;
                    uint32_t b0[NH], b1[NH];
#pragma unroll
                    for (int j = 0; j < NH; ++j) {
                        b0[j] = *reinterpret_cast<const uint32_t*>(hp + j * 64);
                        b1[j] = *reinterpret_cast<const uint32_t*>(hp + j * 64 + (size_t)BP * 8);
                    }
#pragma unroll
                    for (int j = 0; j < NH; ++j) {
                        mma_16816(acc[0][j], afrag[i][0], b0[j], b1[j]);
                        mma_16816(acc[1][j], afrag[i][1], b0[j], b1[j]);
                    }
                }
            }
            // rows are gate rows (unit*4 + gate): scatter them so that the gates of a (unit, sequence) cell are adjacent;
            // ZP = 1 mod 8 keeps the 32 lanes of each store on distinct banks
            float* zq = zpart + (size_t)kq * 8 * ZP * 4;
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int j = 0; j < NH; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int r = m * 16 + b_n + (i >> 1) * 8, n = (nh * NH + j) * 8 + b_k + (i & 1);
                        zq[((size_t)(r >> 2) * ZP + n) * 4 + (r & 3)] = acc[m][j][i];
                    }
        }
        __syncthreads();
        if (tr && tid == 0) tr[1] = clock64();
        // ---- 2. gates: the pairs of a thread are computed side by side (independent chains), stores are predicated
        {
            __half hh[PPT];
#pragma unroll
            for (int q = 0; q < PPT; ++q) {
                float zi = gx[q].x + bias4[q].x, zf = gx[q].y + bias4[q].y, zg = gx[q].z + bias4[q].z,
                      zo = gx[q].w + bias4[q].w;
#pragma unroll
                for (int k = 0; k < kWideKq; ++k) {
                    const float4 zk = *reinterpret_cast<const float4*>(zpart + ((size_t)(k * 8 + gu[q]) * ZP + gn[q]) * 4);
                    zi += zk.x; zf += zk.y; zg += zk.z; zo += zk.w;
                }
                c[q] = sigmoidf_(zf) * c[q] + sigmoidf_(zi) * tanhf_(zg);
                hh[q] = __float2half_rn(sigmoidf_(zo) * tanhf_(c[q]));
            }
#pragma unroll
            for (int q = 0; q < PPT; ++q) {
                if (live[q]) {
                    const int u = u0 + gu[q], n = gn[q];
                    hpub[n * 8 + gu[q]] = __half_as_ushort(hh[q]);
                    if (!a.y_vec) a.y[(size_t)t * a.y_tstride + (size_t)n * a.y_bstride + u] = hh[q];
                    if (s == T - 1) {
                        if (a.hn) a.hn[(size_t)n * H + u] = hh[q];
                        if (a.cn) a.cn[(size_t)n * H + u] = __float2half_rn(c[q]);
                    }
                }
            }
        }
        __syncthreads();
        if (tr && tid == 0) tr[2] = clock64();
        // ---- 3. publish
        if (tid < B) {
            const uint4 v = *reinterpret_cast<const uint4*>(hpub + tid * 8);
            if (s + 1 < T) {
                a.data[((size_t)par * n_cta + cta) * BP + tid] = v;
                // the record is read by the other CTAs' bulk copies (async proxy): the cross-proxy fence sits on the
                // writer side, where it overlaps the release of the flag, instead of in front of every CTA's gather
                asm volatile("fence.proxy.async.global;" ::: "memory");
            }
            if (a.y_vec) *reinterpret_cast<uint4*>(a.y + (size_t)t * a.y_tstride + (size_t)tid * a.y_bstride + u0) = v;
        }
        if (s + 1 == T) break;
        __syncthreads();
        if (tr && tid == 0) tr[3] = clock64();
        const uint32_t tag = a.tag_base + (uint32_t)s + 1u;
        // release: the flag writers fence after the barrier, which covers the record stores of the whole CTA
        if (tid < kBulkFlagCopies)
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.flags + (((size_t)tid * 2 + par) * n_cta + cta) * 32), "r"(tag) : "memory");
        // ---- 4./5. flags and gather, one group of CTAs per warp: the lanes of warp w poll the flags of CTAs
        //      [w*cpw, (w+1)*cpw); as soon as all of them are up, lane 0 hands the group's records (one contiguous
        //      block with the layout of hs) to the bulk-copy engine (no cluster multicast).  A group's copy therefore
        //      starts while slower CTAs are still being waited for, and no CTA-wide barrier sits between flag and copy.
        int timed_out = 0;
        {
            const int c0 = warp * cpw;
            const int c1 = c0 + cpw < n_cta ? c0 + cpw : n_cta;
            if (c0 < n_cta) {   // warp-uniform
                const int j = c0 + lane;
                if (j < c1) {
                    const uint32_t* f = a.flags + (((size_t)(cta % kBulkFlagCopies) * 2 + par) * n_cta + j) * 32;
                    int polls = 0;
                    while (true) {
                        uint32_t v;
                        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                        if (v == tag) break;
                        if (++polls >= a.poll_limit) { timed_out = 1; break; }
                        if ((polls & 1023) == 0 && status_aborted(a.status, a.gen)) { timed_out = 1; break; }
                    }
                    if (timed_out) status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
                    // acquire: one acquire load of the flag just seen (cheaper than a full fence)
                    uint32_t v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                }
                if (tr && tid == 0) tr[4] = clock64();
                const int lost = __any_sync(0xffffffffu, timed_out);   // also orders the lanes' acquires before the copy
                if (lane == 0 && !lost) {
                    const uint32_t off = (uint32_t)c0 * BP * 16u, len = (uint32_t)(c1 - c0) * BP * 16u;
                    pimb200::tc::mbar_expect_tx(gbar_addr, len);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                                 "r"((uint32_t)__cvta_generic_to_shared(hs) + off),
                                 "l"(reinterpret_cast<const unsigned char*>(a.data + (size_t)par * n_cta * BP) + off), "r"(len),
                                 "r"(gbar_addr)
                                 : "memory");
                } else if (lane == 0) {
                    // a flag never came: arrive without a copy, so that the barrier still completes once the copies
                    // the other warps did issue have landed (the CTA waits for them below before it leaves)
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gbar_addr) : "memory");
                }
                if (tr && tid == 0) tr[5] = clock64();
            }
        }
        if (tr && tid == 0) tr[6] = clock64();
        // next step's input-projection term: issued after the fences (a fence waits for loads in flight, and these may
        // come from HBM); consumed after the next tensor-core phase
#pragma unroll
        for (int q = 0; q < PPT; ++q) {
            if (live[q]) {
                const int tn = a.reverse ? t - 1 : t + 1;
                // volatile: the load must issue here, a whole tensor-core phase ahead of its use (left to the
                // scheduler it sinks towards the use to shorten the live range, and its latency lands in the gates)
                const float* gp = a.G + (size_t)tn * a.g_tstride + (size_t)gn[q] * a.g_bstride + (size_t)(u0 + gu[q]) * 4;
                asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];"
                             : "=f"(gx[q].x), "=f"(gx[q].y), "=f"(gx[q].z), "=f"(gx[q].w)
                             : "l"(gp));
            }
        }
        if (!pimb200::tc::mbar_wait(gbar_addr, (uint32_t)(s & 1), reinterpret_cast<const volatile int*>(a.status) + 1, a.gen)) {
            // gave up (a flag or a copy never came, here or in another CTA): before the CTA hands its shared memory
            // back, give the bulk copies it has in flight a bounded chance to land
            for (uint32_t i = 0; i < (1u << 20); ++i)
                if (pimb200::tc::mbar_try_wait(gbar_addr, (uint32_t)(s & 1))) break;
            status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
            timed_out = 1;
        }
        if (__syncthreads_or(timed_out)) return;
        if (tr && tid == 0) tr[7] = clock64();
    }
}

// ---------------------------------------------------------------------------------------------
// two stacked layers as a wavefront (up to 8 sequences, H a multiple of 16 up to 1024): layer A at timestep s and layer
// B at timestep s - 2 in the same step of ONE launch, so a pair of layers costs T + 2 dependent steps instead of 2T.
// It is the wide kernel with its two sequence tiles given to the two layers: slots 0..7 of the exchange records and of
// the hidden-state buffer hold layer A's sequences, slots 8..15 layer B's; the warps of tile half 0 keep layer A's
// W_hh slice in registers, those of tile half 1 layer B's, and the exchange moves both layers' states in the same
// records, flags and bulk copies.  Layer B's input is layer A's output, which every CTA holds after the gather:
// W_ih(B) . h_A is one more product per step, shared by all eight warps (a K quarter of one m-tile each), with the CTA's
// 32 rows of W_ih(B) kept in shared memory (read as mma A fragments, rows padded by 16 bytes: conflict-free); it is made
// a step ahead of its use, under the exchange (see the step loop), and summed by layer B's gate threads next to the
// partials of W_hh(B) . h_B.  Layer A's input projection stays hoisted (G); layer B has none.
// ---------------------------------------------------------------------------------------------
struct WaveArgs {
    const __half* Whh[2];      // packed [4H, H] of layer A, layer B
    const __half* WihB;        // packed [4H, H]: layer B's input matrix
    const float* bias[2];
    const float* G;            // layer A's input-projection terms (fp32)
    long g_tstride, g_bstride;
    const __half* h0[2];
    const __half* c0[2];
    __half* y;                 // layer B's output
    long y_tstride, y_bstride;
    int y_vec;
    __half* hn[2];
    __half* cn[2];
    uint4* data;
    uint32_t* flags;
    uint32_t tag_base;
    int* status;
    int gen;
    int H, T, B;
    int poll_limit;
};

__global__ void __launch_bounds__(kWideThreads, 1) lstm_persistent_wave_kernel(WaveArgs a) {
    constexpr int BP = 16;                           // slots: 8 per layer
    constexpr int ZP = BP + 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, T = a.T, B = a.B;
    const int wp = H + 8;                            // row pitch of the W_ih(B) slice (halves)
    __half* hs = reinterpret_cast<__half*>(smem_raw);                         // [H/8][BP][8]
    float* zpart = reinterpret_cast<float*>(hs + (size_t)BP * H);             // [kWideKq][8 units][ZP][4 gates]
    float* zpart2 = zpart + (size_t)kWideKq * 8 * ZP * 4;                     // same shape: partials of W_ih(B) . h_A
    unsigned short* hpub = reinterpret_cast<unsigned short*>(zpart2 + (size_t)kWideKq * 8 * ZP * 4);  // [BP][8]
    __half* wib = reinterpret_cast<__half*>(hpub + (size_t)BP * 8);           // [32 rows][wp]
    uint64_t* gbar = reinterpret_cast<uint64_t*>(wib + (size_t)32 * wp);
    const uint32_t gbar_addr = (uint32_t)__cvta_generic_to_shared(gbar);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_cta = gridDim.x, cta = blockIdx.x;
    const int u0 = cta * 8;
    const int ktiles = H >> 4;
    const int cpw = (n_cta + kPersistWarps - 1) / kPersistWarps;
    if (tid == 0) {
        pimb200::tc::mbar_init(gbar_addr, (uint32_t)((n_cta + cpw - 1) / cpw));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int kq = warp & (kWideKq - 1), nh = (warp >> 2) & 1;   // nh: the layer whose tile this warp multiplies
    const int b_n = lane >> 2, b_k = (lane & 3) * 2;
    uint32_t afrag[kWideMaxKtw][2][4];
    {
        const __half* wbase = a.Whh[nh] + (size_t)u0 * 4 * H;
#pragma unroll
        for (int i = 0; i < kWideMaxKtw; ++i)
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    afrag[i][m][r] = 0u;
                    if (kWideKq * i + kq < ktiles) {
                        const int row = m * 16 + b_n + (r & 1) * 8;
                        const int k = (kWideKq * i + kq) * 16 + b_k + (r >> 1) * 8;
                        afrag[i][m][r] = __ldg(reinterpret_cast<const uint32_t*>(wbase + (size_t)row * H + k));
                    }
                }
    }
    {
        const int H8 = H >> 3;
        const uint4* src = reinterpret_cast<const uint4*>(a.WihB + (size_t)u0 * 4 * H);
        for (int i = tid; i < 32 * H8; i += kWideThreads) {
            const int r = i / H8, c8 = i - r * H8;
            *reinterpret_cast<uint4*>(wib + (size_t)r * wp + c8 * 8) = __ldg(src + (size_t)r * H8 + c8);
        }
    }
    for (int i = tid; i < BP * H; i += kWideThreads) {
        const int slot = i / H, k = i - slot * H, n = slot & 7;
        const __half* h0 = a.h0[slot >> 3];
        hs[((size_t)(k >> 3) * BP + slot) * 8 + (k & 7)] = (n < B && h0) ? h0[(size_t)n * H + k] : __float2half_rn(0.f);
    }
    for (int i = tid; i < BP * 8; i += kWideThreads) hpub[i] = 0;

    // gate pair of this thread: unit tid / 16, slot tid % 16 (threads 128..255 have none)
    const int gu = tid < 8 * BP ? tid / BP : 0, slot = tid < 8 * BP ? tid % BP : 0;
    const int layer = slot >> 3, gn = slot & 7;
    const bool live = tid < 8 * BP && gn < B;
    float c = 0.f;
    __half hh = __float2half_rn(0.f);
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f), gx = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        const int u = u0 + gu;
        c = a.c0[layer] ? __half2float(a.c0[layer][(size_t)gn * H + u]) : 0.f;
        hh = a.h0[layer] ? a.h0[layer][(size_t)gn * H + u] : __float2half_rn(0.f);
        bias4 = *reinterpret_cast<const float4*>(a.bias[layer] + (size_t)u * 4);
        if (layer == 0) gx = __ldcg(reinterpret_cast<const float4*>(a.G + (size_t)gn * a.g_bstride + (size_t)u * 4));
    }
    __syncthreads();

    // Layer B runs TWO steps behind layer A: its input product W_ih(B) . h_A(t) is then computed from the states already in
    // shared memory right after this CTA has released its flag, while the other CTAs' flags are still on their way (a
    // stretch in which the warps would only spin), and lies ready in zpart2 when layer B's gates need it a step later.
    // One step behind, that product sat between the gather and the gates, on the step's critical path (3.4 us per step).
    for (int s = 0; s <= T + 1; ++s) {
        const int par = s & 1;
        const bool act = layer == 0 ? (s < T) : (s >= 2);      // this thread's layer has a timestep in this step
        const int t = layer == 0 ? s : s - 2;
        // ---- 1. K-partial Z tiles: W_hh . h of the warp's layer
        {
            float acc[2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[m][i] = 0.f;
            const __half* brow = hs + ((size_t)(nh * 8 + b_n)) * 8 + b_k;
#pragma unroll
            for (int i = 0; i < kWideMaxKtw; ++i) {
                if (kWideKq * i + kq < ktiles) {   // warp-uniform
                    const int kt = kWideKq * i + kq;
                    const __half* hp = brow + (size_t)(2 * kt) * BP * 8;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(hp);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(hp + (size_t)BP * 8);
                    mma_16816(acc[0], afrag[i][0], b0, b1);
                    mma_16816(acc[1], afrag[i][1], b0, b1);
                }
            }
            float* zq = zpart + (size_t)kq * 8 * ZP * 4;
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int r = m * 16 + b_n + (i >> 1) * 8, n = nh * 8 + b_k + (i & 1);
                    zq[((size_t)(r >> 2) * ZP + n) * 4 + (r & 3)] = acc[m][i];
                }
        }
        __syncthreads();
        // ---- 2. gates (a layer without a timestep in this step keeps its state)
        if (live) {
            if (act) {
                float zi = gx.x + bias4.x, zf = gx.y + bias4.y, zg = gx.z + bias4.z, zo = gx.w + bias4.w;
#pragma unroll
                for (int k = 0; k < kWideKq; ++k) {
                    const float4 zk = *reinterpret_cast<const float4*>(zpart + ((size_t)(k * 8 + gu) * ZP + slot) * 4);
                    zi += zk.x; zf += zk.y; zg += zk.z; zo += zk.w;
                }
                if (layer == 1) {   // the input product made during the previous step's exchange
#pragma unroll
                    for (int k = 0; k < kWideKq; ++k) {
                        const float4 zk = *reinterpret_cast<const float4*>(zpart2 + ((size_t)(k * 8 + gu) * ZP + slot) * 4);
                        zi += zk.x; zf += zk.y; zg += zk.z; zo += zk.w;
                    }
                }
                c = sigmoidf_(zf) * c + sigmoidf_(zi) * tanhf_(zg);
                hh = __float2half_rn(sigmoidf_(zo) * tanhf_(c));
            }
            const int u = u0 + gu;
            hpub[slot * 8 + gu] = __half_as_ushort(hh);
            if (act) {
                if (layer == 1 && !a.y_vec) a.y[(size_t)t * a.y_tstride + (size_t)gn * a.y_bstride + u] = hh;
                if (t == T - 1) {
                    if (a.hn[layer]) a.hn[layer][(size_t)gn * H + u] = hh;
                    if (a.cn[layer]) a.cn[layer][(size_t)gn * H + u] = __float2half_rn(c);
                }
            }
        }
        __syncthreads();
        // ---- 3. publish both layers' records
        if (tid < BP && (tid & 7) < B) {
            const uint4 v = *reinterpret_cast<const uint4*>(hpub + tid * 8);
            if (s <= T) {
                a.data[((size_t)par * n_cta + cta) * BP + tid] = v;
                asm volatile("fence.proxy.async.global;" ::: "memory");
            }
            if (tid >= 8 && s >= 2 && a.y_vec)
                *reinterpret_cast<uint4*>(a.y + (size_t)(s - 2) * a.y_tstride + (size_t)(tid & 7) * a.y_bstride + u0) = v;
        }
        if (s == T + 1) break;
        __syncthreads();
        const uint32_t tag = a.tag_base + (uint32_t)s + 1u;
        if (tid < kBulkFlagCopies)
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.flags + (((size_t)tid * 2 + par) * n_cta + cta) * 32), "r"(tag) : "memory");
        // ---- 3b. layer B's input product for the NEXT step, from layer A's states still in shared memory (the output of
        //      A's timestep s - 1, which B reaches at step s + 1): warp (kq, nh) takes its K quarter of m-tile nh.  The
        //      barrier behind it keeps every warp's reads of hs ahead of the bulk copies issued below.
        {
            float acc2[4] = {0.f, 0.f, 0.f, 0.f};
            const __half* xrow = hs + (size_t)b_n * 8 + b_k;      // layer A's slots: tile 0
            const __half* arow = wib + (size_t)(nh * 16 + b_n) * wp + b_k;
#pragma unroll 4
            for (int i = 0; i < kWideMaxKtw; ++i) {
                if (kWideKq * i + kq < ktiles) {
                    const int kt = kWideKq * i + kq;
                    const __half* hp = xrow + (size_t)(2 * kt) * BP * 8;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(hp);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(hp + (size_t)BP * 8);
                    const __half* ap = arow + kt * 16;
                    uint32_t af[4];
                    af[0] = *reinterpret_cast<const uint32_t*>(ap);
                    af[1] = *reinterpret_cast<const uint32_t*>(ap + (size_t)8 * wp);
                    af[2] = *reinterpret_cast<const uint32_t*>(ap + 8);
                    af[3] = *reinterpret_cast<const uint32_t*>(ap + (size_t)8 * wp + 8);
                    mma_16816(acc2, af, b0, b1);
                }
            }
            float* zq2 = zpart2 + (size_t)kq * 8 * ZP * 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = nh * 16 + b_n + (i >> 1) * 8, n = 8 + b_k + (i & 1);
                zq2[((size_t)(r >> 2) * ZP + n) * 4 + (r & 3)] = acc2[i];
            }
        }
        __syncthreads();
        // ---- 4./5. flags and gather, one group of CTAs per warp (as in the wide kernel)
        int timed_out = 0;
        {
            const int c0 = warp * cpw;
            const int c1 = c0 + cpw < n_cta ? c0 + cpw : n_cta;
            if (c0 < n_cta) {   // warp-uniform
                const int j = c0 + lane;
                if (j < c1) {
                    const uint32_t* f = a.flags + (((size_t)(cta % kBulkFlagCopies) * 2 + par) * n_cta + j) * 32;
                    int polls = 0;
                    while (true) {
                        uint32_t v;
                        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                        if (v == tag) break;
                        if (++polls >= a.poll_limit) { timed_out = 1; break; }
                        if ((polls & 1023) == 0 && status_aborted(a.status, a.gen)) { timed_out = 1; break; }
                    }
                    if (timed_out) status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
                    uint32_t v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                }
                const int lost = __any_sync(0xffffffffu, timed_out);
                if (lane == 0 && !lost) {
                    const uint32_t off = (uint32_t)c0 * BP * 16u, len = (uint32_t)(c1 - c0) * BP * 16u;
                    pimb200::tc::mbar_expect_tx(gbar_addr, len);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                                 "r"((uint32_t)__cvta_generic_to_shared(hs) + off),
                                 "l"(reinterpret_cast<const unsigned char*>(a.data + (size_t)par * n_cta * BP) + off), "r"(len),
                                 "r"(gbar_addr)
                                 : "memory");
                } else if (lane == 0) {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gbar_addr) : "memory");
                }
            }
        }
        // layer A's input-projection term of the next step
        if (live && layer == 0 && s + 1 < T) {
            const float* gp = a.G + (size_t)(s + 1) * a.g_tstride + (size_t)gn * a.g_bstride + (size_t)(u0 + gu) * 4;
            asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(gx.x), "=f"(gx.y), "=f"(gx.z), "=f"(gx.w) : "l"(gp));
        }
        if (!pimb200::tc::mbar_wait(gbar_addr, (uint32_t)(s & 1), reinterpret_cast<const volatile int*>(a.status) + 1, a.gen)) {
            for (uint32_t i = 0; i < (1u << 20); ++i)
                if (pimb200::tc::mbar_try_wait(gbar_addr, (uint32_t)(s & 1))) break;
            status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
            timed_out = 1;
        }
        if (__syncthreads_or(timed_out)) return;
    }
}

// ---------------------------------------------------------------------------------------------
// pipelined, warp-specialised variant of the register-resident recurrence (1..128 sequences, H <= 1024)
//
// Ownership: CTA (slice c, half b) owns hidden units UPC*c .. UPC*c + UPC - 1 (4*UPC gate rows of W_hh, kept in
// registers as mma A fragments for the whole launch) for the sequences of batch half b.  UPC = 8 gives H/8 CTAs that
// each see every sequence (up to 64, bounded by the shared memory the hidden states of all sequences need); UPC = 16
// with two batch halves gives 2 * H/16 CTAs, each seeing one half of up to 128 sequences: the same number of SMs, half
// as many participants in each half's exchange, twice the sequences per launch.  The halves never interact.
// Within a CTA the sequences are split into NG groups of BPG = 8*NTG that advance independently, and every stage of a
// step has warps of its own, handing over through mbarriers, so that the stages of different groups overlap:
//   * warps 0..7 (tensor) split K eight ways (warp w owns k-tiles w, w+8, ...): wait for the group's gathered hidden
//     states ("full") and for a free partial-sum buffer ("zfree"), multiply, store the K-partials, arrive on "zready".
//     They never wait for the gates: the tensor pipe stays busy with the next group.
//   * warps 8..11 (gates) wait for "zready", sum the eight partials, free the buffer, run the cell update (c stays in
//     fp32 registers for the whole sequence), assemble each sequence's 16-byte records (eight units each) with shuffles,
//     store them (and the y row) and arrive on "done".  The input-projection terms of the next step are fetched into
//     shared memory with cp.async a whole step ahead (they stream from HBM).
//   * warps 12..15 (exchange), one per group: wait for "done", raise this CTA's step flag (release, cumulative over the
//     gate warps' record stores), then poll the flags of the half's CTAs, one flag per lane and chunk of 32 CTAs, and
//     hand each chunk's records to the bulk-copy engine as soon as its flags are up (no cluster multicast); the copies
//     complete on "full".
// The exchange of one group (two L2 round trips plus the skew of the slowest CTA, ~4-5 thousand cycles) runs under the
// arithmetic of the other groups; a step of all groups takes about as long as one group's chain.
// The tensor warpgroups take registers from the others at start-up (setmaxnreg).  Per-sequence arithmetic (k-tile order
// inside a warp's accumulator, order of the eight partial sums) is the same for every UPC / NTG / NG, so a sequence's
// result does not depend on how many sequences share the launch.  Every wait is bounded and ends early once the
// launch's generation appears in the status block.
// ---------------------------------------------------------------------------------------------
constexpr int kPipeTensorWarps = 8;
constexpr int kPipeTensorThreads = kPipeTensorWarps * 32;
constexpr int kPipeGateWarps = 4;
constexpr int kPipeGateThreads = kPipeGateWarps * 32;
constexpr int kPipeThreads = 512;    // 4 warpgroups: 2 tensor, 1 gates, 1 exchange (one warp per group)
constexpr int kPipeKq = 4;           // tensor warp = (K quarter, half of the CTA's gate rows): four partial sums per gate
constexpr int kPipeMh = kPipeTensorWarps / kPipeKq;
constexpr int kPipeKtw = 16;         // k-tiles per tensor warp held in registers (H <= 1024)
constexpr int kPipeMaxGroups = 4;    // one exchange warp per group
constexpr int kPipeMaxHalves = 2;
constexpr int kPipeMaxB = 128;       // sequences per launch: 2 halves x 4 groups x 16
constexpr int kPipeChunk = 32;       // CTAs per gather chunk (one flag per lane)
constexpr int kPipeMaxChunks = 4;    // H <= 1024: at most 128 CTAs per half

struct PipeArgs {
    const __half* Whh;
    const float* bias;
    const float* G;
    long g_tstride, g_bstride;
    const __half* h0;
    const __half* c0;
    __half* y;
    long y_tstride, y_bstride;
    int y_vec;
    __half* hn;
    __half* cn;
    uint4* data;            // [2 parities][halves][NG][H/8 octets][BPG] 16-byte records (the image of a group's hs)
    uint32_t* flags;        // [kBulkFlagCopies][2 parities][kPipeMaxHalves][kPipeMaxGroups][slices] step tags, one per 128-byte line
    uint32_t tag_base;
    int* status;
    int gen;
    int H, T, B;
    int halves;             // batch halves (1 or 2): grid = halves * H / UPC
    int reverse;
    int poll_limit;
    long long* trace;       // optional: 8 clocks per CTA and step
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded mbarrier wait in polls (not clocks); false = gave up or the launch was aborted
__device__ __forceinline__ bool mbar_wait_polls(uint32_t bar, uint32_t parity, const int* status, int gen, int limit) {
    for (int i = 0; i < limit; ++i) {
        if (pimb200::tc::mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255 && status_aborted(status, gen)) return false;
    }
    return false;
}

template <int UPC, int NTG, int NG>
__global__ void __launch_bounds__(kPipeThreads, 1) lstm_persistent_pipe_kernel(PipeArgs a) {
    constexpr int BPG = NTG * 8;                      // sequences per group (padded to whole mma tiles)
    constexpr int MT = UPC / 4;                       // 16-row m-tiles of the CTA's gate rows
    constexpr int OCT = UPC / 8;                      // 16-byte records (unit octets) per sequence and CTA
    static_assert((UPC == 8 || UPC == 16) && BPG <= 32 && NG <= kPipeMaxGroups, "supported shapes");
    constexpr int ZP = BPG + 1;                       // padded sequence pitch of the partial sums
    constexpr int ZBUF = kPipeKq * UPC * ZP * 4;      // floats per partial-sum buffer: [k-quarter][unit][ZP][gate]
    constexpr int MTW = MT / kPipeMh;                 // m-tiles per tensor warp
    static_assert(MT % kPipeMh == 0, "the CTA's gate rows split evenly over the row halves");
    constexpr int SB = (BPG + 15) / 16;               // sequence blocks of 16 per gate thread
    constexpr int CPT = SB * OCT;                     // cells per gate thread and group
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.H, T = a.T;
    __half* hs = reinterpret_cast<__half*>(smem_raw);                                  // [NG][H/8][BPG][8]
    float* zpart = reinterpret_cast<float*>(hs + (size_t)NG * BPG * H);                // [2][ZBUF]
    float4* gxs = reinterpret_cast<float4*>(zpart + 2 * ZBUF);                         // [NG][CPT][128 gate threads]
    uint64_t* bars = reinterpret_cast<uint64_t*>(gxs + (size_t)NG * CPT * kPipeGateThreads);   // full[NG], done[NG], zready[2], zfree[2]
    const uint32_t full0 = (uint32_t)__cvta_generic_to_shared(bars);
    const uint32_t done0 = full0 + 8u * NG;
    const uint32_t zready0 = done0 + 8u * NG;
    const uint32_t zfree0 = zready0 + 16u;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_slices = H / UPC;                     // CTAs per batch half
    const int slice = blockIdx.x % n_slices, half = blockIdx.x / n_slices;
    const int u0 = slice * UPC;
    const int seq0 = half * NG * BPG;                 // first sequence of this half
    const int B = a.B - seq0 < 0 ? 0 : (a.B - seq0 < NG * BPG ? a.B - seq0 : NG * BPG);   // sequences of this half
    const int ktiles = H >> 4;
    const int nchunks = (n_slices + kPipeChunk - 1) / kPipeChunk;
    const int ng_live = (B + BPG - 1) / BPG;          // groups that hold sequences
    // a wait on an mbarrier may take as long as the slowest CTA's flag: same budget as the exchange warps' polls
    const int wait_limit = a.poll_limit < (1 << 27) ? a.poll_limit * 8 : a.poll_limit;
    if (tid == 0) {
        for (int g = 0; g < NG; ++g) {
            pimb200::tc::mbar_init(full0 + 8u * g, (uint32_t)nchunks);          // one arrival (+ bytes) per chunk
            pimb200::tc::mbar_init(done0 + 8u * g, (uint32_t)kPipeGateThreads);
        }
        for (int b = 0; b < 2; ++b) {
            pimb200::tc::mbar_init(zready0 + 8u * b, (uint32_t)kPipeTensorThreads);
            pimb200::tc::mbar_init(zfree0 + 8u * b, (uint32_t)kPipeGateThreads);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // initial hidden states, in the layout of the exchange records: hs[g][j][n][8] = units 8j..8j+7 of sequence g*BPG+n
    for (int i = tid; i < NG * BPG * H; i += kPipeThreads) {
        const int n = i / H, k = i - n * H;
        const int g = n / BPG, nl = n - g * BPG;
        hs[(size_t)g * BPG * H + ((size_t)(k >> 3) * BPG + nl) * 8 + (k & 7)] =
            (n < B && a.h0) ? a.h0[(size_t)(seq0 + n) * H + k] : __float2half_rn(0.f);
    }
    __syncthreads();

    if (warp < kPipeTensorWarps) {
        // ================================ tensor warps ================================
        if (UPC == 16) asm volatile("setmaxnreg.inc.sync.aligned.u32 184;" ::: "memory");
        else asm volatile("setmaxnreg.inc.sync.aligned.u32 136;" ::: "memory");
        const int b_n = lane >> 2, b_k = (lane & 3) * 2;
        // warp = (K quarter kq, row half mh): m-tiles mh*MTW .. of the slice, k-tiles 4i + kq.  Eight K-eighths over all
        // rows would hold the same 128 fragment registers, but then every gate is the sum of eight partials, and the
        // gate warps (one per scheduler, the step's critical resource) spent a third of their phase adding them up
        const int kq = warp % kPipeKq, mh = warp / kPipeKq;
        uint32_t afrag[kPipeKtw][MTW][4];
        {
            const __half* wbase = a.Whh + (size_t)u0 * 4 * H;
#pragma unroll
            for (int i = 0; i < kPipeKtw; ++i)
#pragma unroll
                for (int m = 0; m < MTW; ++m)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        afrag[i][m][r] = 0u;
                        if (kPipeKq * i + kq < ktiles) {
                            const int row = (mh * MTW + m) * 16 + b_n + (r & 1) * 8;
                            const int k = (kPipeKq * i + kq) * 16 + b_k + (r >> 1) * 8;
                            afrag[i][m][r] = __ldg(reinterpret_cast<const uint32_t*>(wbase + (size_t)row * H + k));
                        }
                    }
        }
        int phase = 0;      // group phases executed so far: selects the partial-sum buffer
        bool dead = false;
        for (int s = 0; s < T && !dead; ++s) {
            long long* tr = a.trace ? a.trace + ((size_t)blockIdx.x * T + s) * 8 : nullptr;
            for (int g = 0; g < ng_live; ++g, ++phase) {
                const int zb = phase & 1;
                if (tr && tid == 0 && g == 0) tr[0] = clock64();
                bool ok = true;
                if (s > 0) ok = mbar_wait_polls(full0 + 8u * g, (uint32_t)((s - 1) & 1), a.status, a.gen, wait_limit);
                if (tr && tid == 0 && g == 0) tr[1] = clock64();
                // the partial-sum buffer must have been read by the gate warps (its use two phases ago)
                if (ok && phase >= 2)
                    ok = mbar_wait_polls(zfree0 + 8u * zb, (uint32_t)(((phase >> 1) - 1) & 1), a.status, a.gen, wait_limit);
                if (!ok) { dead = true; break; }
                if (tr && tid == 0 && g == 0) tr[2] = clock64();
                float* zq = zpart + (size_t)zb * ZBUF + (size_t)kq * UPC * ZP * 4;
                float acc[MTW][NTG][4];
#pragma unroll
                for (int m = 0; m < MTW; ++m)
#pragma unroll
                    for (int j = 0; j < NTG; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[m][j][i] = 0.f;
                const __half* brow = hs + (size_t)g * BPG * H + (size_t)b_n * 8 + b_k;
                auto ktile = [&](int i) {
                    const int kt = kPipeKq * i + kq;
                    const __half* hp = brow + (size_t)(2 * kt) * BPG * 8;
                    uint32_t b0[NTG], b1[NTG];
#pragma unroll
                    for (int j = 0; j < NTG; ++j) {
                        b0[j] = *reinterpret_cast<const uint32_t*>(hp + j * 64);
                        b1[j] = *reinterpret_cast<const uint32_t*>(hp + j * 64 + (size_t)BPG * 8);
                    }
#pragma unroll
                    for (int j = 0; j < NTG; ++j)
#pragma unroll
                        for (int m = 0; m < MTW; ++m) mma_16816(acc[m][j], afrag[i][m], b0[j], b1[j]);
                };
                if (ktiles == kPipeKtw * kPipeKq) {
                    // H = 1024: every warp owns sixteen k-tiles; no conditions in the way of scheduling the operand loads
                    // of later k-tiles above the products of earlier ones
#pragma unroll
                    for (int i = 0; i < kPipeKtw; ++i) ktile(i);
                } else {
#pragma unroll
                    for (int i = 0; i < kPipeKtw; ++i)
                        if (kPipeKq * i + kq < ktiles) ktile(i);   // warp-uniform
                }
#pragma unroll
                for (int m = 0; m < MTW; ++m)
#pragma unroll
                    for (int j = 0; j < NTG; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int r = (mh * MTW + m) * 16 + b_n + (i >> 1) * 8, n = j * 8 + b_k + (i & 1);
                            zq[((size_t)(r >> 2) * ZP + n) * 4 + (r & 3)] = acc[m][j][i];
                        }
                mbar_arrive(zready0 + 8u * zb);
                if (tr && tid == 0 && g == 0) tr[3] = clock64();
            }
        }
        if (dead && lane == 0) status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
    } else {
    // the other two warpgroups hand registers over (one instruction per warpgroup, before the roles split up)
    if (UPC == 16) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;" ::: "memory");
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 120;" ::: "memory");
    if (warp < kPipeTensorWarps + kPipeGateWarps) {
        // ================================ gate warps ================================
        // Eight consecutive lanes hold the eight units of one octet of one sequence, so a 16-byte record is assembled
        // with four shuffles and stored by its first lane.  Cell q = (sequence block sb, octet o) of thread gt:
        // unit 8*o + (gt & 7), local sequence gt/8 + 16*sb.
        const int gt = tid - kPipeTensorThreads;          // 0..127
        const int gl = gt & 7;
        float4 bias4[OCT];
#pragma unroll
        for (int o = 0; o < OCT; ++o) bias4[o] = *reinterpret_cast<const float4*>(a.bias + (size_t)(u0 + 8 * o + gl) * 4);
        float c[NG][CPT];
#pragma unroll
        for (int g = 0; g < NG; ++g)
#pragma unroll
            for (int q = 0; q < CPT; ++q) {
                const int o = q % OCT, gn = (gt >> 3) + 16 * (q / OCT), n = g * BPG + gn;
                c[g][q] = (gn < BPG && n < B && a.c0) ? __half2float(a.c0[(size_t)(seq0 + n) * H + u0 + 8 * o + gl]) : 0.f;
            }
        // input-projection terms: fetched with cp.async into this thread's own slots a whole step ahead; one commit
        // group per group phase, so "all but the newest NG - 1 groups" is exactly the phase about to be consumed
        auto prefetch_gx = [&](int g, int t) {
#pragma unroll
            for (int q = 0; q < CPT; ++q) {
                const int o = q % OCT, gn = (gt >> 3) + 16 * (q / OCT), n = g * BPG + gn;
                if (gn < BPG && n < B) {
                    const float* gp = a.G + (size_t)t * a.g_tstride + (size_t)(seq0 + n) * a.g_bstride + (size_t)(u0 + 8 * o + gl) * 4;
                    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(gxs + ((size_t)g * CPT + q) * kPipeGateThreads + gt);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gp) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
#pragma unroll
        for (int g = 0; g < NG; ++g) prefetch_gx(g, a.reverse ? T - 1 : 0);   // (empty commit groups for absent sequences)
        int phase = 0;
        bool dead = false;
        for (int s = 0; s < T && !dead; ++s) {
            const int t = a.reverse ? T - 1 - s : s;
            const int par = s & 1;
            long long* tr = a.trace ? a.trace + ((size_t)blockIdx.x * T + s) * 8 : nullptr;
#pragma unroll
            for (int g = 0; g < NG; ++g) {
                if (g >= ng_live) {   // keep one commit group per group slot, so the wait below stays exact
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    continue;
                }
                const int zb = phase & 1;
                if (!mbar_wait_polls(zready0 + 8u * zb, (uint32_t)((phase >> 1) & 1), a.status, a.gen, wait_limit)) {
                    dead = true;
                    break;
                }
                if (tr && gt == 0 && g == 0) tr[4] = clock64();
                // the cells of a thread are worked side by side (independent chains): partial sums, gate math, then
                // the shuffles and stores
                float z[CPT][4];
                const float* zbp[CPT];
#pragma unroll
                for (int q = 0; q < CPT; ++q) {
                    const int o = q % OCT, gn = (gt >> 3) + 16 * (q / OCT);
                    zbp[q] = zpart + (size_t)zb * ZBUF + ((size_t)(8 * o + gl) * ZP + (gn < BPG ? gn : 0)) * 4;
                    z[q][0] = 0.f; z[q][1] = 0.f; z[q][2] = 0.f; z[q][3] = 0.f;
                }
#pragma unroll
                for (int k = 0; k < kPipeKq; ++k)
#pragma unroll
                    for (int q = 0; q < CPT; ++q) {
                        const float4 zk = *reinterpret_cast<const float4*>(zbp[q] + (size_t)k * UPC * ZP * 4);
                        z[q][0] += zk.x; z[q][1] += zk.y; z[q][2] += zk.z; z[q][3] += zk.w;
                    }
                mbar_arrive(zfree0 + 8u * zb);   // the buffer may be overwritten: its sums are in registers
                asm volatile("cp.async.wait_group %0;" ::"n"(NG - 1) : "memory");   // this phase's input terms have landed
                __half hh[CPT];
#pragma unroll
                for (int q = 0; q < CPT; ++q) {
                    const int o = q % OCT, gn = (gt >> 3) + 16 * (q / OCT), n = g * BPG + gn;
                    float4 gx = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (gn < BPG && n < B) gx = gxs[((size_t)g * CPT + q) * kPipeGateThreads + gt];
                    // order of the additions: input term + bias first, then the sum of the four partials
                    const float zi = (gx.x + bias4[o].x) + z[q][0], zf = (gx.y + bias4[o].y) + z[q][1],
                                zg = (gx.z + bias4[o].z) + z[q][2], zo = (gx.w + bias4[o].w) + z[q][3];
                    c[g][q] = sigmoidf_(zf) * c[g][q] + sigmoidf_(zi) * tanhf_(zg);
                    hh[q] = __float2half_rn(sigmoidf_(zo) * tanhf_(c[g][q]));
                }
#pragma unroll
                for (int q = 0; q < CPT; ++q) {
                    const int o = q % OCT, gn = (gt >> 3) + 16 * (q / OCT), n = g * BPG + gn, u = u0 + 8 * o + gl;
                    const bool live = gn < BPG && n < B;
                    // the octet's record {units 0..7} lands in the lane of unit 0
                    const uint32_t v = (uint32_t)__half_as_ushort(hh[q]);
                    const uint32_t p1 = v | (__shfl_down_sync(0xffffffffu, v, 1, 8) << 16);
                    const uint32_t p2 = __shfl_down_sync(0xffffffffu, p1, 2, 8);
                    const uint32_t q1 = __shfl_down_sync(0xffffffffu, p1, 4, 8);
                    const uint32_t q2 = __shfl_down_sync(0xffffffffu, p2, 4, 8);
                    if (live) {
                        const size_t nn = (size_t)(seq0 + n);
                        if (gl == 0) {
                            const uint4 rec = make_uint4(p1, p2, q1, q2);
                            if (s + 1 < T)
                                a.data[((((size_t)par * a.halves + half) * NG + g) * (H >> 3) + (size_t)slice * OCT + o) * BPG + gn] = rec;
                            if (a.y_vec) *reinterpret_cast<uint4*>(a.y + (size_t)t * a.y_tstride + nn * a.y_bstride + u0 + 8 * o) = rec;
                        }
                        if (!a.y_vec) a.y[(size_t)t * a.y_tstride + nn * a.y_bstride + u] = hh[q];
                        if (s == T - 1) {
                            if (a.hn) a.hn[nn * H + u] = hh[q];
                            if (a.cn) a.cn[nn * H + u] = __float2half_rn(c[g][q]);
                        }
                    }
                }
                // release (CTA scope): the group's exchange warp raises the step flag after this phase completes; its
                // cross-proxy fence and gpu-scope release are cumulative over the record stores above
                mbar_arrive(done0 + 8u * g);
                if (s + 1 < T) prefetch_gx(g, a.reverse ? t - 1 : t + 1);
                else asm volatile("cp.async.commit_group;" ::: "memory");
                if (tr && gt == 0 && g == 0) tr[5] = clock64();
                ++phase;
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (dead && lane == 0) status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
    } else {
        // ================================ exchange warps: warp 12 + g serves group g ================================
        const int g = warp - (kPipeTensorWarps + kPipeGateWarps);
        if (g < ng_live) {
            const int rep = blockIdx.x % kBulkFlagCopies;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(hs + (size_t)g * BPG * H);
            const uint32_t fbar = full0 + 8u * g;
            bool dead = false;
            for (int s = 0; s + 1 < T && !dead; ++s) {
                const int par = s & 1;
                const uint32_t tag = a.tag_base + (uint32_t)s + 1u;
                long long* tr = a.trace ? a.trace + ((size_t)blockIdx.x * T + s) * 8 : nullptr;
                if (!mbar_wait_polls(done0 + 8u * g, (uint32_t)(s & 1), a.status, a.gen, wait_limit)) break;
                // ---- publish: the gate warps' records are out; raise this CTA's step flag in every replica.  The records
                //      are read by the other CTAs' bulk copies (async proxy): the cross-proxy fence sits on the writer
                //      side, here, where its wait for the record stores is the wait the release needs anyway (on the
                //      reader side, in front of the copy, it was measured to cost several thousand cycles per step)
                if (lane < kBulkFlagCopies) asm volatile("fence.proxy.async.global;" ::: "memory");
                if (lane < kBulkFlagCopies)
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(
                                     a.flags + ((((((size_t)lane * 2 + par) * kPipeMaxHalves + half) * kPipeMaxGroups + g) * n_slices + slice) * 32)),
                                 "r"(tag)
                                 : "memory");
                if (tr && lane == 0 && g == 0) tr[6] = clock64();
                // ---- gather: lane l watches slice 32i + l of every chunk i; a chunk's records go to the bulk-copy
                //      engine as soon as its 32 flags are up
                const uint32_t* fbase = a.flags + (((((size_t)rep * 2 + par) * kPipeMaxHalves + half) * kPipeMaxGroups + g) * n_slices) * 32;
                const unsigned char* src =
                    reinterpret_cast<const unsigned char*>(a.data + (((size_t)par * a.halves + half) * NG + g) * (H >> 3) * BPG);
                uint32_t seen = 0;      // bit i: this lane's flag of chunk i carries the tag (or there is no such CTA)
                uint32_t issued = 0;    // bit i: chunk i's copy has been handed to the copy engine (warp-uniform)
#pragma unroll
                for (int i = 0; i < kPipeMaxChunks; ++i)
                    if (i >= nchunks || i * kPipeChunk + lane >= n_slices) seen |= 1u << i;
                for (int i = nchunks; i < kPipeMaxChunks; ++i) issued |= 1u << i;
                constexpr uint32_t all_chunks = (1u << kPipeMaxChunks) - 1u;
                int polls = 0;
                while (issued != all_chunks) {
                    // all of this lane's outstanding flags are loaded before any is looked at: up to four loads in flight
                    uint32_t v[kPipeMaxChunks];
#pragma unroll
                    for (int i = 0; i < kPipeMaxChunks; ++i) {
                        v[i] = tag;
                        if (!(seen >> i & 1u))
                            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];"
                                         : "=r"(v[i])
                                         : "l"(fbase + (size_t)(i * kPipeChunk + lane) * 32)
                                         : "memory");
                    }
#pragma unroll
                    for (int i = 0; i < kPipeMaxChunks; ++i)
                        if (v[i] == tag) seen |= 1u << i;
#pragma unroll
                    for (int i = 0; i < kPipeMaxChunks; ++i) {
                        if ((issued >> i & 1u) || !__all_sync(0xffffffffu, seen >> i & 1u)) continue;
                        // acquire: one acquire load of the flag just seen (polling with acquire loads was measured far
                        // slower); the warp-wide sync orders every lane's acquire before lane 0's copy
                        if (i * kPipeChunk + lane < n_slices) {
                            uint32_t w;
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];"
                                         : "=r"(w)
                                         : "l"(fbase + (size_t)(i * kPipeChunk + lane) * 32)
                                         : "memory");
                        }
                        __syncwarp();
                        if (lane == 0) {
                            const int c0 = i * kPipeChunk, c1 = c0 + kPipeChunk < n_slices ? c0 + kPipeChunk : n_slices;
                            const uint32_t off = (uint32_t)c0 * OCT * BPG * 16u, len = (uint32_t)(c1 - c0) * OCT * BPG * 16u;
                            pimb200::tc::mbar_expect_tx(fbar, len);
                            asm volatile(
                                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst + off),
                                "l"(src + off), "r"(len), "r"(fbar)
                                : "memory");
                        }
                        issued |= 1u << i;
                    }
                    if (issued == all_chunks) break;
                    ++polls;
                    bool lost = polls >= a.poll_limit;
                    if ((polls & 255) == 0 && status_aborted(a.status, a.gen)) lost = true;
                    if (__any_sync(0xffffffffu, lost)) {
                        // a flag never came: arrive without bytes for the chunks not issued, so that the barrier still
                        // completes once the copies that were issued have landed; then leave
                        if (lane == 0) {
                            status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
                            for (int i = 0; i < nchunks; ++i)
                                if (!(issued >> i & 1u)) mbar_arrive(fbar);
                        }
                        dead = true;
                        break;
                    }
                }
                if (tr && lane == 0 && g == 0) tr[7] = clock64();
                if (dead) {
                    // before the CTA hands its shared memory back, give the copies in flight a bounded chance to land
                    for (uint32_t i = 0; i < (1u << 20); ++i)
                        if (pimb200::tc::mbar_try_wait(fbar, (uint32_t)(s & 1))) break;
                }
            }
        }
    }
    }
    __syncthreads();   // no warp leaves (and no shared memory is handed back) before all roles are done
}

// ---------------------------------------------------------------------------------------------
// tcgen05 variant of the batched recurrence (17..64 sequences, H a multiple of 64), opt-in.
//
// The per-step product Z[32 x BP] = W_slice[32 x H] . Hprev[H x BP] runs on the 5th-generation tensor cores: one
// thread issues H/16 tcgen05.mma (kind::f16, M = 128, N = BP, K = 16) per step, the accumulator lives in tensor
// memory, two warps read rows 0..31 back with tcgen05.ld.  Both operands sit in shared memory in the canonical
// K-major 128-byte-swizzled layout, written by ordinary stores / cp.async (the gather writes each exchange record
// straight to its swizzled place).  The instruction's M is 128 but a CTA owns 32 gate rows: the A descriptor of a
// k-block simply runs on into the following shared memory, rows 32..127 of the accumulator are never read.
// Exchange, gates and bounded waits are those of the wide kernel; every exit path frees the tensor memory.
// Measured on B200 at H = 1024, 64 sequences: 14.9 us per step against 8.3 us for the mma.sync kernel of the time
// (4.7 us for today's register-resident one).  With only 32
// useful rows per CTA the instruction is shared-memory-bandwidth bound (each of the 64 MMAs of a step streams the
// full 128-row A window, 6 KB with B), and the swizzled scatter of the gather costs more than the contiguous copy.
// The kernel is therefore opt-in (pimb200_lstm_set_use_tc) and kept as the measured alternative.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {  // byte offset inside a [rows x 64 halves] tile
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(kPersistThreads, 1) lstm_persistent_tc_kernel(BulkArgs a, int BP) {
    using namespace pimb200::tc;
    extern __shared__ unsigned char smem_raw_tc[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw_tc) + 1023) & ~uintptr_t(1023));
    const int H = a.H, T = a.T, B = a.B;
    const int kblocks = H >> 6;
    const int a_kb_bytes = kPersistRows * 128;      // 4 KiB: 32 rows x 64 halves
    const int b_kb_bytes = BP * 128;
    unsigned char* sA = smem;                                           // [kblocks][32 x 128 B]
    unsigned char* sB = sA + (size_t)kblocks * a_kb_bytes;              // [kblocks][BP x 128 B]; also absorbs A's over-read
    float* zbuf = reinterpret_cast<float*>(sB + (size_t)kblocks * b_kb_bytes);   // [32][BP]
    unsigned short* hpub = reinterpret_cast<unsigned short*>(zbuf + (size_t)kPersistRows * BP);  // [BP][8]
    uint64_t* bar = reinterpret_cast<uint64_t*>(hpub + (size_t)BP * 8);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
    const uint32_t bar_addr = smem_u32(bar);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_cta = gridDim.x, cta = blockIdx.x;
    const int u0 = cta * 8;
    const int PPT = (8 * BP + kPersistThreads - 1) / kPersistThreads;  // (unit, sequence) pairs per thread: 1 or 2
    const volatile int* abort_flag = a.status + 1;   // generation of the launch that gave up

    // W_hh slice -> A operand tiles
    {
        const int H8 = H >> 3;
        const uint4* src = reinterpret_cast<const uint4*>(a.Whh + (size_t)u0 * 4 * H);
        for (int i = tid; i < kPersistRows * H8; i += kPersistThreads) {
            const int r = i / H8, c8 = i - r * H8;
            *reinterpret_cast<uint4*>(sA + (size_t)(c8 >> 3) * a_kb_bytes + sw128_offset(r, c8 & 7)) =
                ldg_stream_v4(src + (size_t)r * H8 + c8);
        }
    }
    // h_{-1} -> B operand tiles (rows = sequences; rows >= B stay zero)
    for (int i = tid; i < BP * (H >> 3); i += kPersistThreads) {
        const int n = i / (H >> 3), c8 = i - n * (H >> 3);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (n < B && a.h0) v = *reinterpret_cast<const uint4*>(a.h0 + (size_t)n * H + c8 * 8);
        *reinterpret_cast<uint4*>(sB + (size_t)(c8 >> 3) * b_kb_bytes + sw128_offset(n, c8 & 7)) = v;
    }
    for (int i = tid; i < BP * 8; i += kPersistThreads) hpub[i] = 0;
    if (tid == 0) {
        mbar_init(bar_addr, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int tmem_cols = BP <= 32 ? 32 : 64;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // operand tiles were written by ordinary stores
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // gate pairs of this thread: pair p = tid + q*256 -> unit p / BP, sequence p % BP
    int gu[2], gn[2];
    bool live[2];
    float c[2];
    float4 bias4[2], gx[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int p_ = tid + q * kPersistThreads;
        gu[q] = p_ / BP;
        gn[q] = p_ - gu[q] * BP;
        live[q] = q < PPT && gu[q] < 8 && gn[q] < B;
        c[q] = 0.f;
        bias4[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        gx[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live[q]) {
            const int u = u0 + gu[q];
            c[q] = a.c0 ? __half2float(a.c0[(size_t)gn[q] * H + u]) : 0.f;
            bias4[q] = *reinterpret_cast<const float4*>(a.bias + (size_t)u * 4);
            const int t0 = a.reverse ? T - 1 : 0;
            gx[q] = __ldcg(reinterpret_cast<const float4*>(a.G + (size_t)t0 * a.g_tstride + (size_t)gn[q] * a.g_bstride +
                                                           (size_t)u * 4));
        }
        if (!live[q]) { gu[q] = 0; gn[q] = 0; }   // keeps the unconditional zbuf reads in bounds
    }
    // instruction descriptor: D = f32, A = B = f16, both K-major, N = BP, M = 128
    const uint32_t idesc = (1u << 4) | ((uint32_t)(BP >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    int failed = 0;

    for (int s = 0; s < T; ++s) {
        const int t = a.reverse ? T - 1 - s : s;
        const int par = s & 1;
        long long* tr = a.trace ? a.trace + ((size_t)blockIdx.x * T + s) * 8 : nullptr;
        if (tr && tid == 0) tr[0] = clock64();
        // ---- 1. all of K on the tensor cores, issued by one thread
        if (tid == 32) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int kb = 0; kb < kblocks; ++kb) {
                const uint64_t adesc = make_smem_desc(smem_u32(sA + (size_t)kb * a_kb_bytes));
                const uint64_t bdesc = make_smem_desc(smem_u32(sB + (size_t)kb * b_kb_bytes));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_f16(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(bar_addr);
        }
        // rows 0..31 of the accumulator -> zbuf: warps 0 and 4 own TMEM lanes 0..31, half of the columns each
        if ((warp & 3) == 0 && warp < 8) {
            if (!mbar_wait(bar_addr, (uint32_t)(s & 1), abort_flag, a.gen)) failed = 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (tr && tid == 0) tr[1] = clock64();
            if (!failed) {
                const int half = BP >> 1, c_begin = (warp >> 2) * half;
                for (int c0 = c_begin; c0 < c_begin + half; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + (uint32_t)c0, r);
#pragma unroll
                    for (int q = 0; q < 16; q += 4)
                        *reinterpret_cast<float4*>(zbuf + (size_t)lane * BP + c0 + q) =
                            make_float4(__uint_as_float(r[q]), __uint_as_float(r[q + 1]), __uint_as_float(r[q + 2]),
                                        __uint_as_float(r[q + 3]));
                }
            } else {
                status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        if (__syncthreads_or(failed)) { failed = 1; break; }
        if (tr && tid == 0) tr[2] = clock64();
        // ---- 2. gates
        {
            __half hh[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const float* z = zbuf + (size_t)(gu[q] * 4) * BP + gn[q];
                const float zi = z[0] + gx[q].x + bias4[q].x, zf = z[BP] + gx[q].y + bias4[q].y,
                            zg = z[2 * BP] + gx[q].z + bias4[q].z, zo = z[3 * BP] + gx[q].w + bias4[q].w;
                c[q] = sigmoidf_(zf) * c[q] + sigmoidf_(zi) * tanhf_(zg);
                hh[q] = __float2half_rn(sigmoidf_(zo) * tanhf_(c[q]));
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                if (live[q]) {
                    const int u = u0 + gu[q], n = gn[q];
                    hpub[n * 8 + gu[q]] = __half_as_ushort(hh[q]);
                    if (!a.y_vec) a.y[(size_t)t * a.y_tstride + (size_t)n * a.y_bstride + u] = hh[q];
                    if (s == T - 1) {
                        if (a.hn) a.hn[(size_t)n * H + u] = hh[q];
                        if (a.cn) a.cn[(size_t)n * H + u] = __float2half_rn(c[q]);
                    }
                }
            }
        }
        __syncthreads();
        if (tr && tid == 0) tr[3] = clock64();
        // ---- 3. publish
        if (tid < B) {
            const uint4 v = *reinterpret_cast<const uint4*>(hpub + tid * 8);
            if (s + 1 < T) {
                a.data[((size_t)par * n_cta + cta) * BP + tid] = v;
                __threadfence();
            }
            if (a.y_vec) *reinterpret_cast<uint4*>(a.y + (size_t)t * a.y_tstride + (size_t)tid * a.y_bstride + u0) = v;
        }
        if (s + 1 == T) break;
        __syncthreads();
        if (tr && tid == 0) tr[4] = clock64();
        const uint32_t tag = a.tag_base + (uint32_t)s + 1u;
        if (tid < kBulkFlagCopies)
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(a.flags + (((size_t)tid * 2 + par) * n_cta + cta) * 32), "r"(tag) : "memory");
        // ---- 4. flags
        int timed_out = 0;
        if (tid < n_cta) {
            const uint32_t* f = a.flags + (((size_t)(cta % kBulkFlagCopies) * 2 + par) * n_cta + tid) * 32;
            int polls = 0;
            while (true) {
                uint32_t v;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                if (v == tag) break;
                if (++polls >= a.poll_limit) { timed_out = 1; break; }
                if ((polls & 1023) == 0 && status_aborted(a.status, a.gen)) { timed_out = 1; break; }
            }
            if (timed_out) status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
            __threadfence();
        }
        if (__syncthreads_or(timed_out)) { failed = 1; break; }
        if (tr && tid == 0) tr[5] = clock64();
        // ---- 5. gather: record (cta j, sequence n) = 16-byte chunk (j & 7) of row n in k-block j >> 3
        {
            const uint4* src = a.data + (size_t)par * n_cta * BP;
            const uint32_t dst0 = smem_u32(sB);
            const int items = n_cta * BP;
            for (int i = tid; i < items; i += kPersistThreads) {
                const int j = i / BP, n = i - j * BP;
                const uint32_t dst = dst0 + (uint32_t)(j >> 3) * (uint32_t)b_kb_bytes + sw128_offset(n, j & 7);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + i) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                if (live[q]) {
                    const int tn = a.reverse ? t - 1 : t + 1;
                    gx[q] = __ldcg(reinterpret_cast<const float4*>(a.G + (size_t)tn * a.g_tstride +
                                                                   (size_t)gn[q] * a.g_bstride + (size_t)(u0 + gu[q]) * 4));
                }
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads these tiles next
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tr && tid == 0) tr[6] = clock64();
    }
    // common exit: nobody may still use the tensor memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct pimb200_lstm {
    int L = 0, D = 1, I = 0, H = 0, has_biases = 0, device = 0;
    int variant = PIMB200_LSTM_AUTO;
    int sm_count = kNumSmB200;
    int max_smem_optin = 0;
    std::vector<__half*> w_ih, w_hh;  // per (l*D+d), packed
    std::vector<float*> bias;         // per (l*D+d), packed fp32
    // workspace, grown on demand
    float* G = nullptr;
    size_t G_cap = 0;
    __half* ybuf[2] = {nullptr, nullptr};
    size_t y_cap[2] = {0, 0};
    float* cstate = nullptr;
    size_t c_cap = 0;
    // packed input on the lock-step kernels: lengths, packed row offsets, padded input copy, one direction's run output
    int* pk_lens = nullptr;
    size_t pk_lens_cap = 0;
    long* pk_row0 = nullptr;
    size_t pk_row0_cap = 0;
    __half* pk_x = nullptr;
    size_t pk_x_cap = 0;
    __half* pk_run = nullptr;
    size_t pk_run_cap = 0;
    int packed_lockstep = 1;   // 0: packed input runs timestep by timestep on the streamed kernels
    int wavefront = 1;         // 1: stacked layers of up to 8 sequences run in pairs, one step apart, in one launch
    uint4* xchg = nullptr;  // [kXchgCopies][2][kXchgWords]
    uint4* bulk_data = nullptr;      // batched variant: [2][n_cta][32] records
    uint32_t* bulk_flags = nullptr;  // [2][n_cta]
    uint32_t bulk_tag = 0;
    int* d_status = nullptr;         // {sticky error code, generation of the launch that gave up}
    int launch_gen = 0;              // generation handed to the last persistent launch (never 0)
    uint32_t tag_counter = 0;
    int poll_limit = kPersistPollLimit;
    int use_tc = 0;        // 1 = tcgen05 recurrence for 17..64 sequences (measured slower than mma.sync here: opt-in)
    int bulk_wide = 2;     // 2 = pipelined kernel for 33..128 sequences, wide kernel below (default), 3 = pipelined kernel
                           // for every batch size, 1 = wide kernel (exchange on the compute warps, up to 64 sequences),
                           // 0 = K-split kernel with W_hh in shared memory (up to 32 sequences)
    int pipe_group_size = 0;   // sequences per group of the pipelined kernel: 0 = choose by batch size, else 8, 16 or 32
    int xchg_copies = 4;   // measured: 4 replicas, words 128 B apart (one sequence) or 32 B apart (several)
    int xchg_stride = 0;   // 0 = choose by batch size
    long long* trace = nullptr;  // diagnostics buffer supplied through pimb200_lstm_set_trace (not owned)
    // optional timing of the recurrence launches (CUDA events on the launching stream)
    bool prof = false;
    std::vector<cudaEvent_t> prof_ev;   // pairs: begin, end
    size_t prof_used = 0;
    double prof_bytes = 0.0;            // algorithmic W_hh bytes of the timed launches
    std::mutex mu;
};

static void prof_mark(pimb200_lstm* h, cudaStream_t st) {
    if (h->prof_used == h->prof_ev.size()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return;
        h->prof_ev.push_back(e);
    }
    cudaEventRecord(h->prof_ev[h->prof_used++], st);
}

static int next_gen(pimb200_lstm* h) {
    if (++h->launch_gen == 0) h->launch_gen = 1;
    return h->launch_gen;
}

static int in_size(const pimb200_lstm* h, int l) { return l == 0 ? h->I : h->D * h->H; }

extern "C" int pimb200_lstm_destroy(pimb200_lstm* h) {
    if (!h) return PIMB200_OK;
    cudaSetDevice(h->device);
    for (auto p : h->w_ih) cudaFree(p);
    for (auto p : h->w_hh) cudaFree(p);
    for (auto p : h->bias) cudaFree(p);
    cudaFree(h->G);
    cudaFree(h->pk_lens);
    cudaFree(h->pk_row0);
    cudaFree(h->pk_x);
    cudaFree(h->pk_run);
    cudaFree(h->ybuf[0]);
    cudaFree(h->ybuf[1]);
    cudaFree(h->cstate);
    cudaFree(h->xchg);
    cudaFree(h->bulk_data);
    cudaFree(h->bulk_flags);
    cudaFree(h->d_status);
    for (auto e : h->prof_ev) cudaEventDestroy(e);
    delete h;
    return PIMB200_OK;
}

extern "C" int pimb200_lstm_create(const void* const* params, int n_params, int num_layers, int bidirectional,
                                   int input_size, int hidden_size, int has_biases, pimb200_lstm** out) {
    if (!params || !out || num_layers <= 0 || input_size <= 0 || hidden_size <= 0) return PIMB200_ERR_BAD_ARG;
    const int D = bidirectional ? 2 : 1;
    const int per = has_biases ? 4 : 2;
    if (n_params != per * D * num_layers) return PIMB200_ERR_BAD_ARG;
    for (int i = 0; i < n_params; ++i)
        if (!params[i]) return PIMB200_ERR_BAD_ARG;
    pimb200_lstm* h = new pimb200_lstm();
    h->L = num_layers; h->D = D; h->I = input_size; h->H = hidden_size; h->has_biases = has_biases ? 1 : 0;
    int rc = PIMB200_OK;
    auto fail = [&](int code) { pimb200_lstm_destroy(h); return code; };
    if (cudaGetDevice(&h->device) != cudaSuccess) return fail(PIMB200_ERR_LAUNCH);
    cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, h->device);
    cudaDeviceGetAttribute(&h->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, h->device);
    const int H = hidden_size;
    for (int l = 0; l < num_layers; ++l) {
        for (int d = 0; d < D; ++d) {
            const int Il = in_size(h, l);
            const void* const* p = params + (size_t)(l * D + d) * per;
            __half *wi = nullptr, *wh = nullptr;
            float* bs = nullptr;
            if (cudaMalloc(&wi, (size_t)4 * H * Il * 2) != cudaSuccess) return fail(PIMB200_ERR_NO_MEMORY);
            h->w_ih.push_back(wi);
            if (cudaMalloc(&wh, (size_t)4 * H * H * 2) != cudaSuccess) return fail(PIMB200_ERR_NO_MEMORY);
            h->w_hh.push_back(wh);
            if (cudaMalloc(&bs, (size_t)4 * H * 4) != cudaSuccess) return fail(PIMB200_ERR_NO_MEMORY);
            h->bias.push_back(bs);
            lstm_pack_matrix_kernel<<<296, 256>>>(static_cast<const __half*>(p[0]), wi, H, Il);
            lstm_pack_matrix_kernel<<<296, 256>>>(static_cast<const __half*>(p[1]), wh, H, H);
            lstm_pack_bias_kernel<<<ceil_div(4 * H, 256), 256>>>(
                has_biases ? static_cast<const __half*>(p[2]) : nullptr,
                has_biases ? static_cast<const __half*>(p[3]) : nullptr, bs, H);
        }
    }
    if (cudaMalloc(&h->xchg, kXchgBytes) != cudaSuccess) return fail(PIMB200_ERR_NO_MEMORY);
    if (cudaMalloc(&h->d_status, 8) != cudaSuccess) return fail(PIMB200_ERR_NO_MEMORY);
    cudaMemset(h->xchg, 0, kXchgBytes);
    {
        const size_t ncta = (size_t)ceil_div(H, 8);
        // records of both parities: the pipelined kernel's layout (up to kPipeMaxB sequences) is the largest
        if (cudaMalloc(&h->bulk_data, 2 * ncta * kPipeMaxB * 16) != cudaSuccess) return fail(PIMB200_ERR_NO_MEMORY);
        const size_t flag_bytes = (size_t)kBulkFlagCopies * 2 * kPipeMaxHalves * kPipeMaxGroups * ncta * 128;   // the pipelined kernel's layout is the largest
        if (cudaMalloc(&h->bulk_flags, flag_bytes) != cudaSuccess) return fail(PIMB200_ERR_NO_MEMORY);
        cudaMemset(h->bulk_flags, 0, flag_bytes);
    }
    cudaMemset(h->d_status, 0, 8);
    if ((rc = cuda_status(cudaDeviceSynchronize())) != PIMB200_OK) return fail(rc);
    *out = h;
    return PIMB200_OK;
}

extern "C" int pimb200_lstm_set_variant(pimb200_lstm* h, int variant) {
    if (!h || variant < 0 || variant > 3) return PIMB200_ERR_BAD_ARG;
    h->variant = variant;
    return PIMB200_OK;
}

// test hook: shrink the bounded wait so a withheld arrival is detected quickly (not part of the public header's
// stable surface, but exported so host-side fault tests can reach it)
extern "C" int pimb200_lstm_set_poll_limit(pimb200_lstm* h, int limit) {
    if (!h || limit <= 0) return PIMB200_ERR_BAD_ARG;
    h->poll_limit = limit;
    return PIMB200_OK;
}

// Timing hook used by the benchmark: when enabled, every recurrence (all T steps of one layer/direction) is
// bracketed by CUDA events on the launching stream.  read() synchronises those events and returns the summed
// device time, the number of recurrences and their algorithmic W_hh bytes (T * 4H*H * 2 each), then clears.
extern "C" int pimb200_lstm_profile_enable(pimb200_lstm* h, int enable) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lk(h->mu);
    h->prof = enable != 0;
    h->prof_used = 0;
    h->prof_bytes = 0.0;
    return PIMB200_OK;
}
extern "C" int pimb200_lstm_profile_read(pimb200_lstm* h, double* total_ms, long* recurrences, double* bytes) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lk(h->mu);
    double ms = 0.0;
    for (size_t i = 0; i + 1 < h->prof_used; i += 2) {
        PIMB200_CUDA_TRY(cudaEventSynchronize(h->prof_ev[i + 1]));
        float t = 0.f;
        PIMB200_CUDA_TRY(cudaEventElapsedTime(&t, h->prof_ev[i], h->prof_ev[i + 1]));
        ms += t;
    }
    if (total_ms) *total_ms = ms;
    if (recurrences) *recurrences = (long)(h->prof_used / 2);
    if (bytes) *bytes = h->prof_bytes;
    h->prof_used = 0;
    h->prof_bytes = 0.0;
    return PIMB200_OK;
}

// Diagnostics: a device buffer of n_cta * T * 8 int64 that the persistent kernel fills with per-step clocks.
// Diagnostics / tuning: how many replicas of the exchange buffer the persistent kernel publishes into.
extern "C" int pimb200_lstm_set_exchange_copies(pimb200_lstm* h, int copies) {
    if (!h || copies < 1 || copies > kXchgCopies) return PIMB200_ERR_BAD_ARG;
    h->xchg_copies = copies;
    return PIMB200_OK;
}
// A/B switch: 0 = never use the tcgen05 recurrence kernel.
extern "C" int pimb200_lstm_set_use_tc(pimb200_lstm* h, int on) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    h->use_tc = on ? 1 : 0;
    return PIMB200_OK;
}
// A/B switch between the two batched kernels for 17..32 sequences (the wide one also takes 33..64).
extern "C" int pimb200_lstm_set_bulk_wide(pimb200_lstm* h, int on) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    h->bulk_wide = on < 0 ? 0 : (on > 3 ? 3 : on);
    return PIMB200_OK;
}
// A/B switch: 0 runs stacked layers one after the other, 1 (default) pairs of layers as a wavefront (up to 8 sequences).
extern "C" int pimb200_lstm_set_wavefront(pimb200_lstm* h, int on) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    h->wavefront = on ? 1 : 0;
    return PIMB200_OK;
}
// A/B switch: 0 runs packed input timestep by timestep on the streamed kernels, 1 (default) as a padded lock-step batch.
extern "C" int pimb200_lstm_set_packed_lockstep(pimb200_lstm* h, int on) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    h->packed_lockstep = on ? 1 : 0;
    return PIMB200_OK;
}
// Tuning switch of the pipelined kernel: sequences per independently advancing group (8, 16 or 32; 0 = by batch size).
extern "C" int pimb200_lstm_set_pipe_group_size(pimb200_lstm* h, int seqs) {
    if (!h || (seqs != 0 && seqs != 8 && seqs != 16 && seqs != 32)) return PIMB200_ERR_BAD_ARG;
    h->pipe_group_size = seqs;
    return PIMB200_OK;
}
extern "C" int pimb200_lstm_set_exchange_stride(pimb200_lstm* h, int stride16) {
    if (!h || stride16 < 1 || stride16 > kXchgMaxStride) return PIMB200_ERR_BAD_ARG;
    h->xchg_stride = stride16;
    h->tag_counter = 0xffffu;  // forces a fresh tag generation (zeroed buffer) at the next launch
    return PIMB200_OK;
}
extern "C" int pimb200_lstm_set_trace(pimb200_lstm* h, long long* device_buffer) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    h->trace = device_buffer;
    return PIMB200_OK;
}

extern "C" int pimb200_lstm_last_status(pimb200_lstm* h) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    int v = 0;
    PIMB200_CUDA_TRY(cudaMemcpy(&v, h->d_status, 4, cudaMemcpyDeviceToHost));
    if (v != 0) PIMB200_CUDA_TRY(cudaMemset(h->d_status, 0, 4));
    return v;
}

template <typename T>
static int grow(T** p, size_t* cap, size_t need_elems) {
    if (*cap >= need_elems) return PIMB200_OK;
    PIMB200_CUDA_TRY(cudaDeviceSynchronize());  // earlier launches may still use the old block
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    PIMB200_CUDA_TRY(cudaMalloc(p, need_elems * sizeof(T)));
    *cap = need_elems;
    return PIMB200_OK;
}

static size_t wide_smem(int H, int nt) {
    const int BP = nt * 8;
    return (size_t)BP * H * 2 + (size_t)kWideKq * 8 * (BP + 1) * 16 + (size_t)BP * 16 + 16;
}
static size_t pipe_smem(int H, int upc, int ntg, int ng) {
    const int BPG = ntg * 8, cpt = ((BPG + 15) / 16) * (upc / 8);
    return (size_t)ng * BPG * H * 2 + (size_t)2 * kPipeKq * upc * (BPG + 1) * 16 +
           (size_t)ng * cpt * kPipeGateThreads * 16 + (size_t)(2 * ng + 4) * 8 + 16;
}
static size_t tc_smem(int H, int BP) {
    return (size_t)(H / 64) * (kPersistRows * 128 + BP * 128) + (size_t)kPersistRows * BP * 4 + (size_t)BP * 16 + 64 + 1024;
}
static size_t bulk_smem(int H, int nt) {
    const int BP = nt * 8;
    return (size_t)kPersistRows * (H + 8) * 2 + (size_t)BP * (H + 8) * 2 + (size_t)kPersistWarps * kPersistRows * BP * 4 +
           (size_t)BP * 16;
}
struct PersistPlan { bool ok; int U, ncta, threads; size_t smem; };
static size_t persist_smem(int H, int B) {
    return (size_t)kPersistRows * (H + 8) * 2 + (size_t)2 * B * (H + 8) * 2 +
           (size_t)kPersistWarps * kPersistRows * 8 * 4 + 128;
}
static PersistPlan plan_persistent(const pimb200_lstm* h) {
    PersistPlan p{false, 0, 0, 0, 0};
    const int H = h->H;
    if (H % 16 != 0) return p;                       // K is consumed in m16n8k16 tiles
    const int U = ceil_div(H, h->sm_count);
    if (U > kUnitsPerWord) return p;                 // one 16-byte exchange word per CTA
    p.U = U;
    p.ncta = ceil_div(H, U);
    if (p.ncta > kXchgWords || p.ncta > kPersistThreads) return p;
    p.threads = kPersistThreads;
    p.smem = persist_smem(H, kPersistMaxB);
    if ((int)persist_smem(H, 1) > h->max_smem_optin) return p;
    p.ok = true;
    return p;
}

// one (layer, direction) recurrence over a padded batch or a packed sequence
struct SeqLayout {
    int T, B;                       // B = batch_sizes[0] for packed input
    const int64_t* batch_sizes;     // NULL for padded input
    std::vector<long> row0;         // packed: first row of timestep t
};

static int run_recurrence(pimb200_lstm* h, int ld, const SeqLayout& sq, bool reverse, const float* G, long g_tstride,
                          long g_bstride, const __half* h0, const __half* c0, __half* y, long y_tstride,
                          long y_bstride, __half* hn, __half* cn, cudaStream_t st) {
    const int H = h->H, T = sq.T, B = sq.B;
    const bool packed = sq.batch_sizes != nullptr;
    bool use_persistent = false;
    PersistPlan pp = plan_persistent(h);
    const bool fits = pp.ok && B <= kPersistMaxB && !packed && (int)persist_smem(H, B) <= h->max_smem_optin;
    const int nt = B <= 8 ? 1 : (B <= 16 ? 2 : (B <= 32 ? 4 : 8));
    // 2..64 sequences: the register-resident kernel (2.8 / 3.4 / 4.7 us per step at 16 / 32 / 64 sequences against
    // 4.3 / 5.8 for the K-split one at 16 / 32)
    // (the wide kernel keeps its W_hh slice in registers: H at most 1024)
    const bool wide_ok = (H % 16 == 0) && H <= 16 * kWideKq * kWideMaxKtw;
    const bool wide = wide_ok && h->bulk_wide >= 1;
    const int wnt = nt < 2 ? 2 : nt;   // the wide kernel's smallest instance takes 16 sequences
    const size_t bsmem = wide ? wide_smem(H, wnt) : bulk_smem(H, nt);
    const bool bulk_fits = (H % 16 == 0) && (H / 8 <= h->sm_count) && (H / 8 <= kPersistThreads) && B >= (wide ? 1 : 2) &&
                           B <= (h->bulk_wide ? kBulkMaxB : 32) && (nt <= 4 || wide) && !packed && (int)bsmem <= h->max_smem_optin;
    // tensor-core (tcgen05) recurrence: 17..64 sequences, H a multiple of 64
    const int tc_bp = B <= 32 ? 32 : 64;   // accumulator columns; two warps read half of them each, 16 at a time
    // the A descriptor of the last k-block runs 12 KiB past the weight tiles: the B tiles behind them must cover that
    const bool tc_fits = h->use_tc && (H % 64 == 0) && (H / 8 <= h->sm_count) && (H / 8 <= kPersistThreads) && B > 16 &&
                         B <= kBulkMaxB && !packed && (size_t)(H / 64) * tc_bp * 128 >= 12288 &&
                         (int)tc_smem(H, tc_bp) <= h->max_smem_optin;
    if (tc_fits && (h->variant == PIMB200_LSTM_PERSISTENT || (h->variant == PIMB200_LSTM_AUTO && T >= 8))) {
        BulkArgs a;
        a.Whh = h->w_hh[ld]; a.bias = h->bias[ld]; a.G = G; a.g_tstride = g_tstride; a.g_bstride = g_bstride;
        a.h0 = h0; a.c0 = c0; a.y = y; a.y_tstride = y_tstride; a.y_bstride = y_bstride; a.hn = hn; a.cn = cn;
        a.y_vec = (aligned16(y) && y_tstride % 8 == 0 && y_bstride % 8 == 0) ? 1 : 0;
        a.data = h->bulk_data; a.flags = h->bulk_flags; a.tag_base = h->bulk_tag; a.status = h->d_status; a.gen = next_gen(h);
        a.H = H; a.T = T; a.B = B; a.reverse = reverse ? 1 : 0; a.poll_limit = h->poll_limit;
        a.trace = h->trace;
        h->bulk_tag += (uint32_t)T + 1u;
        int bp = tc_bp;
        const size_t smem = tc_smem(H, bp);
        PIMB200_CUDA_TRY(cudaFuncSetAttribute(lstm_persistent_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        void* kargs[] = {&a, &bp};
        if (h->prof) prof_mark(h, st);
        PIMB200_CUDA_TRY(cudaLaunchCooperativeKernel((const void*)lstm_persistent_tc_kernel, dim3(H / 8),
                                                     dim3(kPersistThreads), kargs, smem, st));
        if (h->prof) {
            prof_mark(h, st);
            h->prof_bytes += (double)T * 4.0 * H * H * 2.0;
        }
        return PIMB200_OK;
    }
    // pipelined register-resident recurrence: the default for 33..128 lock-step sequences (below that a step is mostly
    // exchange latency with little to overlap it with, and the wide kernel's shorter chain wins); 65..128 sequences run
    // as two batch halves on CTAs of 16 hidden units each
    const bool pipe_shape = wide_ok && !packed && B <= kPipeMaxB && (H / 8 <= h->sm_count) && (B <= 64 || H % 16 == 0);
    const bool pipe_wanted = h->bulk_wide >= 2 && (B > 32 || h->bulk_wide >= 3);
    if (pipe_shape && pipe_wanted && !tc_fits &&
        (h->variant == PIMB200_LSTM_PERSISTENT || (h->variant == PIMB200_LSTM_AUTO && T >= 8))) {
        const int upc = B > 64 ? 16 : 8, halves = B > 64 ? 2 : 1;
        const int b_half = halves == 2 ? 64 : B;   // sequences the first half holds
        // sequences per group (8, 16 or 32) and the smallest instantiated group count (at most 4) that holds a half
        int bpg = h->pipe_group_size;
        if (bpg == 0) bpg = 16;
        if (bpg * kPipeMaxGroups < b_half) bpg = 16;
        if (upc == 16) bpg = 16;
        const int need = ceil_div(b_half, bpg);
        const int ng = need <= 1 ? 1 : (need <= 2 ? 2 : 4);
        const int ntg = bpg / 8;
        const size_t smem = pipe_smem(H, upc, ntg, ng);
        if ((int)smem <= h->max_smem_optin) {
            PipeArgs a;
            a.Whh = h->w_hh[ld]; a.bias = h->bias[ld]; a.G = G; a.g_tstride = g_tstride; a.g_bstride = g_bstride;
            a.h0 = h0; a.c0 = c0; a.y = y; a.y_tstride = y_tstride; a.y_bstride = y_bstride; a.hn = hn; a.cn = cn;
            a.y_vec = (aligned16(y) && y_tstride % 8 == 0 && y_bstride % 8 == 0) ? 1 : 0;
            a.data = h->bulk_data; a.flags = h->bulk_flags; a.tag_base = h->bulk_tag; a.status = h->d_status; a.gen = next_gen(h);
            a.H = H; a.T = T; a.B = B; a.halves = halves; a.reverse = reverse ? 1 : 0; a.poll_limit = h->poll_limit;
            a.trace = h->trace;
            h->bulk_tag += (uint32_t)T + 1u;
            const void* fn = nullptr;
            if (upc == 16) {
                fn = (const void*)lstm_persistent_pipe_kernel<16, 2, 4>;
            } else {
                switch (ntg * 16 + ng) {
                    case 1 * 16 + 1: fn = (const void*)lstm_persistent_pipe_kernel<8, 1, 1>; break;
                    case 1 * 16 + 2: fn = (const void*)lstm_persistent_pipe_kernel<8, 1, 2>; break;
                    case 1 * 16 + 4: fn = (const void*)lstm_persistent_pipe_kernel<8, 1, 4>; break;
                    case 2 * 16 + 1: fn = (const void*)lstm_persistent_pipe_kernel<8, 2, 1>; break;
                    case 2 * 16 + 2: fn = (const void*)lstm_persistent_pipe_kernel<8, 2, 2>; break;
                    case 2 * 16 + 4: fn = (const void*)lstm_persistent_pipe_kernel<8, 2, 4>; break;
                    case 4 * 16 + 1: fn = (const void*)lstm_persistent_pipe_kernel<8, 4, 1>; break;
                    default: fn = (const void*)lstm_persistent_pipe_kernel<8, 4, 2>; break;
                }
            }
            PIMB200_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            void* kargs[] = {&a};
            if (h->prof) prof_mark(h, st);
            PIMB200_CUDA_TRY(cudaLaunchCooperativeKernel(fn, dim3(halves * H / upc), dim3(kPipeThreads), kargs, smem, st));
            if (h->prof) {
                prof_mark(h, st);
                // each batch half is a recurrence of its own on its own CTAs, with its own register-resident copy of W_hh
                h->prof_bytes += (double)halves * T * 4.0 * H * H * 2.0;
            }
            return PIMB200_OK;
        }
    }
    if (B > kBulkMaxB && !packed && h->variant != PIMB200_LSTM_STREAMED && h->variant != PIMB200_LSTM_AUTO)
        return PIMB200_ERR_UNSUPPORTED;   // a persistent variant was requested for a batch only the pipelined kernel takes
    bool use_bulk = false;
    if (h->variant == PIMB200_LSTM_PERSISTENT) {
        if (!fits && !bulk_fits) return PIMB200_ERR_UNSUPPORTED;
        use_bulk = bulk_fits;
        use_persistent = !use_bulk;
    } else if (h->variant == PIMB200_LSTM_PERSISTENT_TAGGED) {
        if (!fits) return PIMB200_ERR_UNSUPPORTED;
        use_persistent = true;
    } else if (h->variant == PIMB200_LSTM_AUTO) {
        use_bulk = bulk_fits && T >= 8;
        use_persistent = !use_bulk && fits && T >= 8;
    }
    if (use_bulk) {
        BulkArgs a;
        a.Whh = h->w_hh[ld]; a.bias = h->bias[ld]; a.G = G; a.g_tstride = g_tstride; a.g_bstride = g_bstride;
        a.h0 = h0; a.c0 = c0; a.y = y; a.y_tstride = y_tstride; a.y_bstride = y_bstride; a.hn = hn; a.cn = cn;
        a.y_vec = (aligned16(y) && y_tstride % 8 == 0 && y_bstride % 8 == 0) ? 1 : 0;
        a.data = h->bulk_data; a.flags = h->bulk_flags; a.tag_base = h->bulk_tag; a.status = h->d_status; a.gen = next_gen(h);
        a.H = H; a.T = T; a.B = B; a.reverse = reverse ? 1 : 0; a.poll_limit = h->poll_limit;
        a.trace = h->trace;
        h->bulk_tag += (uint32_t)T + 1u;
        const void* fn = wide ? (wnt == 2   ? (const void*)lstm_persistent_wide_kernel<2>
                                 : wnt == 4 ? (const void*)lstm_persistent_wide_kernel<4>
                                            : (const void*)lstm_persistent_wide_kernel<8>)
                              : (nt == 1   ? (const void*)lstm_persistent_bulk_kernel<1>
                                 : nt == 2 ? (const void*)lstm_persistent_bulk_kernel<2>
                                           : (const void*)lstm_persistent_bulk_kernel<4>);
        const size_t smem = bsmem;
        PIMB200_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        void* kargs[] = {&a};
        if (h->prof) prof_mark(h, st);
        PIMB200_CUDA_TRY(cudaLaunchCooperativeKernel(fn, dim3(H / 8), dim3(wide ? kWideThreads : kPersistThreads), kargs, smem, st));
        if (h->prof) {
            prof_mark(h, st);
            h->prof_bytes += (double)T * 4.0 * H * H * 2.0;
        }
        return PIMB200_OK;
    }
    if (use_persistent) {
        PersistArgs a;
        a.Whh = h->w_hh[ld]; a.bias = h->bias[ld]; a.G = G; a.g_tstride = g_tstride; a.g_bstride = g_bstride;
        a.h0 = h0; a.c0 = c0; a.y = y; a.y_tstride = y_tstride; a.y_bstride = y_bstride; a.hn = hn; a.cn = cn;
        a.B = B;
        pp.smem = persist_smem(H, B);
        a.xchg = h->xchg; a.tag_base = h->tag_counter; a.status = h->d_status; a.gen = next_gen(h);
        a.H = H; a.T = T; a.U = pp.U; a.reverse = reverse ? 1 : 0; a.poll_limit = h->poll_limit;
        a.trace = h->trace;
        a.copies = h->xchg_copies;
        a.wstride = h->xchg_stride > 0 ? h->xchg_stride : (B == 1 ? 8 : 2);
        // step tags are 16 bits wide: start a fresh generation (zeroed buffer, tags from 1) before they could wrap
        // onto a stale word left by an earlier launch
        if ((h->tag_counter & 0xffffu) + (uint32_t)T + 1u > 0xffffu) {
            PIMB200_CUDA_TRY(cudaMemsetAsync(h->xchg, 0, kXchgBytes, st));
            h->tag_counter = 0;
            a.tag_base = 0;
        }
        h->tag_counter += (uint32_t)T + 1u;
        const void* fn = (const void*)lstm_persistent_kernel;
        PIMB200_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pp.smem));
        void* kargs[] = {&a};
        if (h->prof) prof_mark(h, st);
        PIMB200_CUDA_TRY(cudaLaunchCooperativeKernel(fn, dim3(pp.ncta), dim3(pp.threads), kargs, pp.smem, st));
        if (h->prof) {
            prof_mark(h, st);
            h->prof_bytes += (double)T * 4.0 * H * H * 2.0;
        }
        return PIMB200_OK;
    }
    // streamed
    int rc = grow(&h->cstate, &h->c_cap, (size_t)B * H);
    if (rc != PIMB200_OK) return rc;
    lstm_init_c_kernel<<<ceil_div(B * H, 256), 256, 0, st>>>(h->cstate, c0, B * H);
    const bool vec = (H % 8 == 0) && aligned16(h0 ? h0 : h->w_hh[ld]) && aligned16(y) && (y_bstride % 8 == 0) &&
                     (y_tstride % 8 == 0);
    if (h->prof) prof_mark(h, st);
    for (int s = 0; s < T; ++s) {
        const int t = reverse ? T - 1 - s : s;
        const int tp = reverse ? t + 1 : t - 1;  // timestep that produced h_prev
        StepArgs a;
        a.Whh = h->w_hh[ld]; a.bias = h->bias[ld]; a.H = H; a.h0 = h0; a.c = h->cstate;
        a.hp_bstride = y_bstride; a.ho_bstride = y_bstride; a.g_bstride = g_bstride;
        if (packed) {
            a.B = (int)sq.batch_sizes[t];
            a.G = G + (size_t)sq.row0[t] * g_tstride;
            a.hout = y + (size_t)sq.row0[t] * y_tstride;
            if (s == 0) { a.n_prev = 0; a.hprev_seq = nullptr; }
            else { a.n_prev = (int)std::min<int64_t>(sq.batch_sizes[tp], a.B); a.hprev_seq = y + (size_t)sq.row0[tp] * y_tstride; }
            // forward: a sequence's last active step is its final state, so refresh hn/cn every step
            const bool write_final = reverse ? (s == T - 1) : true;
            a.hn = write_final ? hn : nullptr;
            a.cn = write_final ? cn : nullptr;
        } else {
            a.B = B;
            a.G = G + (size_t)t * g_tstride;
            a.hout = y + (size_t)t * y_tstride;
            if (s == 0) { a.n_prev = 0; a.hprev_seq = nullptr; }
            else { a.n_prev = B; a.hprev_seq = y + (size_t)tp * y_tstride; }
            a.hn = (s == T - 1) ? hn : nullptr;
            a.cn = (s == T - 1) ? cn : nullptr;
        }
        if (a.B <= 0) continue;
        const int grid = ceil_div(H, 8);
        if (vec) {
            if (a.B == 1) lstm_step_kernel<1, true><<<grid, 256, 0, st>>>(a);
            else if (a.B == 2) lstm_step_kernel<2, true><<<grid, 256, 0, st>>>(a);
            else lstm_step_kernel<4, true><<<grid, 256, 0, st>>>(a);
        } else {
            if (a.B == 1) lstm_step_kernel<1, false><<<grid, 256, 0, st>>>(a);
            else lstm_step_kernel<4, false><<<grid, 256, 0, st>>>(a);
        }
    }
    if (h->prof) {
        prof_mark(h, st);
        h->prof_bytes += (double)T * 4.0 * H * H * 2.0;
    }
    return launch_status();
}

// ---------------------------------------------------------------------------------------------
// packed sequences on the lock-step recurrences
//
// A packed batch (sequences sorted by decreasing length, timestep t holds its first batch_sizes[t] sequences) runs as a
// padded [T, B] batch through the same persistent kernels as padded input:
//   * the input is scattered into padded time-major rows (zeros behind each sequence); the backward direction gets
//     every sequence reversed on its own, so it too is a forward recurrence that starts at the sequence's first step
//     with the caller's initial state, and its outputs are reversed back when they are stored;
//   * behind a sequence's end the gate terms of its input and forget gates are set to -1e4 / +1e4: sigmoid gives exactly
//     0 and 1, the cell state stays frozen, so the kernel's c_n is the state after the sequence's own last step;
//     h_n is the output row of that step, picked up when the outputs are stored.
// ---------------------------------------------------------------------------------------------
struct PackedMeta {
    const int* lens;       // [B] device
    const long* row0;      // [T] device: first packed row of timestep t
};

// dst[t, b, :] (padded, row t*B+b, `w` halves) <- row (ts, b) of src, ts = reverse ? len_b-1-t : t; zeros for t >= len_b.
// src is packed (row0[ts] + b) when src_packed, else padded (ts*B + b), rows src_ld halves apart.
__global__ void lstm_to_padded_kernel(const __half* __restrict__ src, long src_ld, int src_packed, __half* __restrict__ dst,
                                      PackedMeta m, int T, int B, int w, int reverse) {
    const long row = blockIdx.x;
    const int t = (int)(row / B), b = (int)(row % B);
    const int len = m.lens[b];
    __half* d = dst + row * (long)w;
    if (t >= len) {
        for (int c = threadIdx.x; c < w; c += blockDim.x) d[c] = __float2half_rn(0.f);
        return;
    }
    const int ts = reverse ? len - 1 - t : t;
    const __half* sp = src + (src_packed ? (m.row0[ts] + b) : ((long)ts * B + b)) * src_ld;
    for (int c = threadIdx.x; c < w; c += blockDim.x) d[c] = sp[c];
}

// Behind each sequence's end: input gate off, forget gate on, the other two terms zero (packed gate order i, f, g, o).
__global__ void lstm_freeze_gates_kernel(float* __restrict__ G, PackedMeta m, int T, int B, int H) {
    const long row = blockIdx.x;
    const int t = (int)(row / B), b = (int)(row % B);
    if (t < m.lens[b]) return;
    float4* g = reinterpret_cast<float4*>(G + row * 4L * H);
    for (int u = threadIdx.x; u < H; u += blockDim.x) g[u] = make_float4(-1.0e4f, 1.0e4f, 0.f, 0.f);
}

// Stores the outputs of one direction's padded run (src [T, B, H], contiguous): row (t, b) of the run is timestep
// ts = reverse ? len_b-1-t : t of sequence b.  Destination: packed rows (row0[ts] + b) or padded rows (ts*B + b), dst_ld
// halves apart, at column offset col; padded destinations get zeros behind the sequence.  The run's row len_b-1 is h_n.
__global__ void lstm_from_padded_kernel(const __half* __restrict__ src, __half* __restrict__ dst, long dst_ld, int dst_packed,
                                        int col, __half* __restrict__ hn, PackedMeta m, int T, int B, int H, int reverse) {
    const long row = blockIdx.x;
    const int t = (int)(row / B), b = (int)(row % B);
    const int len = m.lens[b];
    if (t >= len) {
        if (!dst_packed) {
            __half* d = dst + ((long)t * B + b) * dst_ld + col;
            for (int c = threadIdx.x; c < H; c += blockDim.x) d[c] = __float2half_rn(0.f);
        }
        return;
    }
    const int ts = reverse ? len - 1 - t : t;
    const __half* sp = src + row * (long)H;
    __half* d = dst + (dst_packed ? (m.row0[ts] + b) : ((long)ts * B + b)) * dst_ld + col;
    for (int c = threadIdx.x; c < H; c += blockDim.x) d[c] = sp[c];
    if (hn && t == len - 1) {
        __half* hp = hn + (long)b * H;
        for (int c = threadIdx.x; c < H; c += blockDim.x) hp[c] = sp[c];
    }
}

static int run_recurrence(pimb200_lstm* h, int ld, const SeqLayout& sq, bool reverse, const float* G, long g_tstride,
                          long g_bstride, const __half* h0, const __half* c0, __half* y, long y_tstride,
                          long y_bstride, __half* hn, __half* cn, cudaStream_t st);

static int lstm_forward_packed_lockstep(pimb200_lstm* h, const __half* data, const SeqLayout& sq, const __half* h0,
                                        const __half* c0, __half* y, __half* hn, __half* cn, cudaStream_t st) {
    const int H = h->H, D = h->D, L = h->L, T = sq.T, B = sq.B;
    const long prow = (long)T * B;
    int rc;
    // sequence lengths and packed row offsets, uploaded once per call
    std::vector<int> lens(B, 0);
    for (int t = 0; t < T; ++t)
        for (int b = 0; b < (int)sq.batch_sizes[t]; ++b) lens[b] = t + 1;
    if ((rc = grow(&h->pk_lens, &h->pk_lens_cap, (size_t)B)) != PIMB200_OK) return rc;
    if ((rc = grow(&h->pk_row0, &h->pk_row0_cap, (size_t)T)) != PIMB200_OK) return rc;
    PIMB200_CUDA_TRY(cudaMemcpyAsync(h->pk_lens, lens.data(), sizeof(int) * B, cudaMemcpyHostToDevice, st));
    PIMB200_CUDA_TRY(cudaMemcpyAsync(h->pk_row0, sq.row0.data(), sizeof(long) * T, cudaMemcpyHostToDevice, st));
    // (a copy from pageable host memory returns once the source has been staged, so the vectors may go out of scope)
    const PackedMeta meta{h->pk_lens, h->pk_row0};
    int max_in = h->I;
    if (L > 1 && D * H > max_in) max_in = D * H;
    if ((rc = grow(&h->pk_x, &h->pk_x_cap, (size_t)prow * max_in)) != PIMB200_OK) return rc;
    if ((rc = grow(&h->pk_run, &h->pk_run_cap, (size_t)prow * H)) != PIMB200_OK) return rc;
    if ((rc = grow(&h->G, &h->G_cap, (size_t)prow * 4 * H)) != PIMB200_OK) return rc;
    if (L > 1 && (rc = grow(&h->ybuf[0], &h->y_cap[0], (size_t)prow * D * H)) != PIMB200_OK) return rc;
    if (L > 2 && (rc = grow(&h->ybuf[1], &h->y_cap[1], (size_t)prow * D * H)) != PIMB200_OK) return rc;
    SeqLayout padded;
    padded.T = T; padded.B = B; padded.batch_sizes = nullptr;
    const unsigned grid = (unsigned)prow;
    for (int l = 0; l < L; ++l) {
        const int Il = in_size(h, l);
        const bool first = (l == 0), last = (l == L - 1);
        const __half* Xin = first ? data : h->ybuf[(l - 1) & 1];      // packed rows (layer 0) or padded rows
        __half* Yout = last ? y : h->ybuf[l & 1];
        for (int d = 0; d < D; ++d) {
            const int ld = l * D + d;
            const __half* X = Xin;
            if (first || d == 1) {   // padded (and, for the backward direction, per-sequence reversed) copy of the input
                lstm_to_padded_kernel<<<grid, 128, 0, st>>>(Xin, Il, first ? 1 : 0, h->pk_x, meta, T, B, Il, d);
                X = h->pk_x;
            }
            if ((rc = launch_gemm_wx(h->w_ih[ld], X, nullptr, h->G, 4 * H, Il, (int)prow, Il, 4 * H, PIMB200_ACT_NONE, 1, st)) !=
                PIMB200_OK)
                return rc;
            lstm_freeze_gates_kernel<<<grid, 128, 0, st>>>(h->G, meta, T, B, H);
            const __half* h0_ld = h0 ? h0 + (size_t)ld * B * H : nullptr;
            const __half* c0_ld = c0 ? c0 + (size_t)ld * B * H : nullptr;
            __half* cn_ld = cn ? cn + (size_t)ld * B * H : nullptr;
            if ((rc = run_recurrence(h, ld, padded, false, h->G, (long)B * 4 * H, 4L * H, h0_ld, c0_ld, h->pk_run, (long)B * H,
                                     (long)H, nullptr, cn_ld, st)) != PIMB200_OK)
                return rc;
            lstm_from_padded_kernel<<<grid, 128, 0, st>>>(h->pk_run, Yout, (long)D * H, last ? 1 : 0, d * H,
                                                          hn ? hn + (size_t)ld * B * H : nullptr, meta, T, B, H, d);
            if ((rc = launch_status()) != PIMB200_OK) return rc;
        }
    }
    return PIMB200_OK;
}

static size_t wave_smem(int H) {
    return (size_t)16 * H * 2 + (size_t)2 * kWideKq * 8 * 17 * 16 + (size_t)16 * 16 + (size_t)32 * (H + 8) * 2 + 16;
}
// Layers l and l + 1 (one direction) as a wavefront: true when the shape is the wave kernel's
static bool wave_fits(const pimb200_lstm* h, int l, int T, int B, bool packed) {
    const int H = h->H;
    return h->wavefront && !packed && h->D == 1 && l + 1 < h->L && T >= 8 && B >= 1 && B <= 8 && H % 16 == 0 &&
           H <= 16 * kWideKq * kWideMaxKtw && H / 8 <= h->sm_count && H / 8 <= kPersistThreads && h->bulk_wide >= 1 &&
           (h->variant == PIMB200_LSTM_AUTO || h->variant == PIMB200_LSTM_PERSISTENT) && (int)wave_smem(H) <= h->max_smem_optin;
}
static int run_wave(pimb200_lstm* h, int l, int T, int B, const float* G, long g_tstride, long g_bstride, const __half* h0,
                    const __half* c0, __half* y, long y_tstride, long y_bstride, __half* hn, __half* cn, cudaStream_t st) {
    const int H = h->H;
    WaveArgs a;
    for (int k = 0; k < 2; ++k) {
        const size_t off = (size_t)(l + k) * B * H;
        a.Whh[k] = h->w_hh[l + k];
        a.bias[k] = h->bias[l + k];
        a.h0[k] = h0 ? h0 + off : nullptr;
        a.c0[k] = c0 ? c0 + off : nullptr;
        a.hn[k] = hn ? hn + off : nullptr;
        a.cn[k] = cn ? cn + off : nullptr;
    }
    a.WihB = h->w_ih[l + 1];
    a.G = G; a.g_tstride = g_tstride; a.g_bstride = g_bstride;
    a.y = y; a.y_tstride = y_tstride; a.y_bstride = y_bstride;
    a.y_vec = (aligned16(y) && y_tstride % 8 == 0 && y_bstride % 8 == 0) ? 1 : 0;
    a.data = h->bulk_data; a.flags = h->bulk_flags; a.tag_base = h->bulk_tag; a.status = h->d_status; a.gen = next_gen(h);
    a.H = H; a.T = T; a.B = B; a.poll_limit = h->poll_limit;
    h->bulk_tag += (uint32_t)T + 3u;
    const size_t smem = wave_smem(H);
    const void* fn = (const void*)lstm_persistent_wave_kernel;
    PIMB200_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    void* kargs[] = {&a};
    if (h->prof) prof_mark(h, st);
    PIMB200_CUDA_TRY(cudaLaunchCooperativeKernel(fn, dim3(H / 8), dim3(kWideThreads), kargs, smem, st));
    if (h->prof) {
        prof_mark(h, st);
        h->prof_bytes += 2.0 * T * 4.0 * H * H * 2.0;   // two layers' W_hh per timestep
    }
    return PIMB200_OK;
}

static int lstm_forward_impl(pimb200_lstm* h, const __half* x, const SeqLayout& sq, const __half* h0,
                             const __half* c0, __half* y, __half* hn, __half* cn, int batch_first,
                             cudaStream_t st) {
    std::lock_guard<std::mutex> lk(h->mu);
    const int H = h->H, D = h->D, L = h->L, T = sq.T, B = sq.B;
    const bool packed = sq.batch_sizes != nullptr;
    long rows = 0;  // rows of the flattened [rows, features] activations
    if (packed) rows = sq.row0[T - 1] + (long)sq.batch_sizes[T - 1];
    else rows = (long)T * B;
    int rc;
    // packed input of several steps: as a padded lock-step batch on the persistent recurrences (needs the 128-bit GEMM
    // path for the padded rows; the streamed kernels below take every other case)
    if (packed && h->packed_lockstep && h->variant != PIMB200_LSTM_STREAMED && T > 1 && H % 16 == 0 && B <= kPipeMaxB)
        return lstm_forward_packed_lockstep(h, x, sq, h0, c0, y, hn, cn, st);
    // decode form: seq_len 1, every extent a multiple of 8 and 16-byte aligned -> one fused cell launch per layer
    bool cell = !packed && T == 1 && h->variant != PIMB200_LSTM_PERSISTENT && h->variant != PIMB200_LSTM_PERSISTENT_TAGGED &&
                H % 8 == 0 && h->I % 8 == 0 && aligned16(x) && aligned16(y) && (!h0 || aligned16(h0));
    const bool cell_gemm = cell && B >= kCellGemmMinB;   // lock-step decode of many sequences: products as GEMMs
    if (cell_gemm && (rc = grow(&h->G, &h->G_cap, (size_t)2 * B * 4 * H)) != PIMB200_OK) return rc;
    if (!cell && (rc = grow(&h->G, &h->G_cap, (size_t)rows * 4 * H)) != PIMB200_OK) return rc;
    if (L > 1 && (rc = grow(&h->ybuf[0], &h->y_cap[0], (size_t)rows * D * H)) != PIMB200_OK) return rc;
    if (L > 2 && (rc = grow(&h->ybuf[1], &h->y_cap[1], (size_t)rows * D * H)) != PIMB200_OK) return rc;
    if (cell) {
        for (int l = 0; l < L; ++l) {
            const bool last = (l == L - 1);
            const __half* X = l == 0 ? x : h->ybuf[(l - 1) & 1];
            __half* Y = last ? y : h->ybuf[l & 1];
            for (int d = 0; d < D; ++d) {
                const int ld = l * D + d;
                CellArgs a;
                a.Wih = h->w_ih[ld]; a.Whh = h->w_hh[ld]; a.bias = h->bias[ld];
                a.x = X; a.x_bstride = in_size(h, l);
                a.h0 = h0 ? h0 + (size_t)ld * B * H : nullptr;
                a.c0 = c0 ? c0 + (size_t)ld * B * H : nullptr;
                a.y = Y + (size_t)d * H; a.y_bstride = (long)D * H;
                a.hn = hn ? hn + (size_t)ld * B * H : nullptr;
                a.cn = cn ? cn + (size_t)ld * B * H : nullptr;
                a.I = in_size(h, l); a.H = H; a.B = B;
                if (cell_gemm) {
                    float* Gx = h->G;
                    float* Gh = a.h0 ? h->G + (size_t)B * 4 * H : nullptr;
                    if ((rc = launch_gemm_wx(a.Wih, a.x, nullptr, Gx, 4 * H, a.I, B, (int)a.x_bstride, 4 * H, PIMB200_ACT_NONE, 1,
                                             st)) != PIMB200_OK)
                        return rc;
                    if (Gh && (rc = launch_gemm_wx(a.Whh, a.h0, nullptr, Gh, 4 * H, H, B, H, 4 * H, PIMB200_ACT_NONE, 1, st)) !=
                                  PIMB200_OK)
                        return rc;
                    CellPointArgs pa{Gx, Gh, a.bias, a.c0, a.y, a.y_bstride, a.hn, a.cn, H, B, nullptr, 0};
                    lstm_cell_point_kernel<<<ceil_div(B * H, 256), 256, 0, st>>>(pa);
                    if ((rc = launch_status()) != PIMB200_OK) return rc;
                    continue;
                }
                if (B == 1) lstm_cell_kernel<1><<<ceil_div(H, 8), 256, 0, st>>>(a);
                else lstm_cell_kernel<4><<<ceil_div(H, 8), 256, 0, st>>>(a);
                if ((rc = launch_status()) != PIMB200_OK) return rc;
            }
        }
        return PIMB200_OK;
    }
    for (int l = 0; l < L; ++l) {
        const int Il = in_size(h, l);
        const bool first = (l == 0), last = (l == L - 1);
        const __half* X = first ? x : h->ybuf[(l - 1) & 1];
        __half* Y = last ? y : h->ybuf[l & 1];
        // row index of (t, b): user layout on the outermost tensors, time-major in between
        long in_t, in_b, out_t, out_b;
        if (packed) { in_t = 1; in_b = 1; out_t = 1; out_b = 1; }  // row = row0[t] + b
        else {
            in_t = (first && batch_first) ? 1 : B;  in_b = (first && batch_first) ? T : 1;
            out_t = (last && batch_first) ? 1 : B;  out_b = (last && batch_first) ? T : 1;
        }
        for (int d = 0; d < D; ++d) {
            const int ld = l * D + d;
            // A batch-first input is projected into time-major rows when the tensor-core path allows it: the terms
            // the recurrence needs in one step then sit side by side (with the input's own order the 64 sequences of
            // a step lie megabytes apart, one page each, and the per-step loads miss the TLB)
            long g_t = in_t, g_b = in_b;
            rc = PIMB200_ERR_UNSUPPORTED;
            if (first && batch_first && !packed && B > 1 && T > 1) {
                rc = launch_gemm_wx_time_major(h->w_ih[ld], X, h->G, 4 * H, Il, (int)rows, Il, 4 * H, B, st);
                if (rc == PIMB200_OK) { g_t = B; g_b = 1; }
            }
            if (rc == PIMB200_ERR_UNSUPPORTED)
                rc = launch_gemm_wx(h->w_ih[ld], X, nullptr, h->G, 4 * H, Il, (int)rows, Il, 4 * H, PIMB200_ACT_NONE, 1,
                                    st);
            if (rc != PIMB200_OK) return rc;
            if (wave_fits(h, l, T, B, packed)) {
                // layers l and l + 1 in one launch, one step apart; the pair's output is layer l + 1's
                const bool last2 = (l + 1 == L - 1);
                __half* Y2 = last2 ? y : h->ybuf[(l + 1) & 1];
                const long o_t = (last2 && batch_first) ? 1 : B, o_b = (last2 && batch_first) ? T : 1;
                rc = run_wave(h, l, T, B, h->G, g_t * 4 * H, g_b * 4 * H, h0, c0, Y2, o_t * (long)H, o_b * (long)H, hn, cn, st);
                if (rc != PIMB200_OK) return rc;
                ++l;   // the second layer of the pair is done
                break;
            }
            const __half* h0_ld = h0 ? h0 + (size_t)ld * B * H : nullptr;
            const __half* c0_ld = c0 ? c0 + (size_t)ld * B * H : nullptr;
            __half* hn_ld = hn ? hn + (size_t)ld * B * H : nullptr;
            __half* cn_ld = cn ? cn + (size_t)ld * B * H : nullptr;
            rc = run_recurrence(h, ld, sq, d == 1, h->G, g_t * 4 * H, g_b * 4 * H, h0_ld, c0_ld,
                                Y + (size_t)d * H, out_t * (long)D * H, out_b * (long)D * H, hn_ld, cn_ld, st);
            if (rc != PIMB200_OK) return rc;
        }
    }
    return PIMB200_OK;
}

extern "C" int pimb200_lstm_forward(pimb200_lstm* h, const void* x, int T, int B, const void* h0, const void* c0,
                                    void* y, void* hn, void* cn, int batch_first, void* stream) {
    if (!h || !x || !y || T <= 0 || B <= 0) return PIMB200_ERR_BAD_ARG;
    SeqLayout sq;
    sq.T = T; sq.B = B; sq.batch_sizes = nullptr;
    return lstm_forward_impl(h, static_cast<const __half*>(x), sq, static_cast<const __half*>(h0),
                             static_cast<const __half*>(c0), static_cast<__half*>(y), static_cast<__half*>(hn),
                             static_cast<__half*>(cn), batch_first ? 1 : 0, static_cast<cudaStream_t>(stream));
}

// Decode step of a one-layer, one-direction handle for B >= 8 sequences with strided rows: x rows x_ld halves apart, the
// output (optionally h + residual) written to rows y_ld halves apart, e.g. straight into one half of the next layer's
// concatenated input.
extern "C" int pimb200_lstm_forward_step(pimb200_lstm* h, const void* x, long x_ld, int B, const void* h0, const void* c0,
                                         void* y, long y_ld, void* hn, void* cn, const void* residual, long residual_ld,
                                         void* stream) {
    if (!h || !x || !y || B <= 0) return PIMB200_ERR_BAD_ARG;
    const int H = h->H, I = h->I;
    if (x_ld < I || y_ld < H || (residual && residual_ld < H)) return PIMB200_ERR_BAD_ARG;
    if (h->L != 1 || h->D != 1 || B < kCellGemmMinB || H % 8 != 0 || I % 8 != 0 || x_ld % 8 != 0 || !aligned16(x) ||
        (h0 && !aligned16(h0)))
        return PIMB200_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(h->mu);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    if ((rc = grow(&h->G, &h->G_cap, (size_t)2 * B * 4 * H)) != PIMB200_OK) return rc;
    float* Gx = h->G;
    float* Gh = h0 ? h->G + (size_t)B * 4 * H : nullptr;
    if ((rc = launch_gemm_wx(h->w_ih[0], static_cast<const __half*>(x), nullptr, Gx, 4 * H, I, B, (int)x_ld, 4 * H,
                             PIMB200_ACT_NONE, 1, st)) != PIMB200_OK)
        return rc;
    if (Gh && (rc = launch_gemm_wx(h->w_hh[0], static_cast<const __half*>(h0), nullptr, Gh, 4 * H, H, B, H, 4 * H,
                                   PIMB200_ACT_NONE, 1, st)) != PIMB200_OK)
        return rc;
    CellPointArgs pa{Gx, Gh, h->bias[0], static_cast<const __half*>(c0), static_cast<__half*>(y), y_ld,
                     static_cast<__half*>(hn), static_cast<__half*>(cn), H, B, static_cast<const __half*>(residual), residual_ld};
    lstm_cell_point_kernel<<<ceil_div(B * H, 256), 256, 0, st>>>(pa);
    return launch_status();
}

extern "C" int pimb200_lstm_forward_packed(pimb200_lstm* h, const void* data, const int64_t* batch_sizes, int T,
                                           const void* h0, const void* c0, void* y, void* hn, void* cn,
                                           void* stream) {
    if (!h || !data || !y || !batch_sizes || T <= 0) return PIMB200_ERR_BAD_ARG;
    SeqLayout sq;
    sq.T = T; sq.B = (int)batch_sizes[0]; sq.batch_sizes = batch_sizes;
    if (sq.B <= 0) return PIMB200_ERR_BAD_ARG;
    sq.row0.resize(T);
    long acc = 0;
    for (int t = 0; t < T; ++t) {
        if (batch_sizes[t] <= 0 || (t > 0 && batch_sizes[t] > batch_sizes[t - 1])) return PIMB200_ERR_BAD_ARG;
        sq.row0[t] = acc;
        acc += (long)batch_sizes[t];
    }
    return lstm_forward_impl(h, static_cast<const __half*>(data), sq, static_cast<const __half*>(h0),
                             static_cast<const __half*>(c0), static_cast<__half*>(y), static_cast<__half*>(hn),
                             static_cast<__half*>(cn), 0, static_cast<cudaStream_t>(stream));
}
