// Batched-stream linear layer for few activation rows:  Y[J, N] = act(X[J, K] . W[N, K]^T + bias[N]),  J <= 32.
//
// This is the batch 8 / 32 form of the batch-1 GEMV (several utterance streams sharing one weight matrix, or the
// branches of a MULTISTREAM node): the arithmetic intensity is J flop per weight byte, far below the ridge, so the
// bound is the one pass over W from HBM, exactly as for the GEMV.  A 128-row tcgen05 tile per CTA leaves most SMs
// without work at N = 4096 (32 CTAs) and costs a fixed pipeline set-up; here every SM streams W instead:
//   * a CTA owns 16 or 32 weight rows (one or two 16-row tiles), its 8 warps split the tiles and K between them
//     (32 rows x 4 K-quarters for N >= 2048: one CTA per SM at N = 4096, 64 KB of W per SM in flight, and the two
//     tiles of a K-quarter share their X loads through L1; 16 rows x 8 K-eighths below that, for more CTAs);
//   * a warp reads its W rows with 128-bit loads that bypass L1, 8 consecutive k per thread and row, and uses them
//     directly as mma.sync m16n8k16 A fragments: the contraction index is only a summation order, so the k positions
//     a thread holds (k0 + 8t .. k0 + 8t + 7 of rows g and g + 8) are fed as the fragment's "2t, 2t+1, 2t+8, 2t+9"
//     slots of two products, and the B fragment (X, read through L1: it is small and shared by all CTAs) is taken
//     from the same k positions.  No shared-memory staging, no shuffles;
//   * the K-partials meet in shared memory; the CTA's rows x J outputs get bias, activation and the fp16 (or fp32) store.
#include "common.cuh"

namespace pimb200 {

namespace {
constexpr int kSkinnyWarps = 8;
constexpr int kSkinnyThreads = kSkinnyWarps * 32;
constexpr int kSkinnyRows = 16;
constexpr int kSkinnyMaxJ = 32;

__device__ __forceinline__ void mma16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkinnyArgs {
    const __half* W;      // [N, K] row-major
    const __half* X;      // [J, ldx]
    const __half* bias;   // [N] or NULL
    void* Y;              // [J, ldy] fp16 or fp32
    int N, K, J, ldx, ldy, act, y_is_f32;
};

template <int NT, int MTC>   // n-tiles of 8 activation rows; 16-row weight tiles per CTA (1 or 2)
__global__ void __launch_bounds__(kSkinnyThreads) gemm_skinny_kernel(SkinnyArgs a) {
    constexpr int KS = kSkinnyWarps / MTC;   // K splits
    constexpr int ROWS = MTC * kSkinnyRows;
    __shared__ float part[KS][ROWS][NT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int mt = warp % MTC, ks = warp / MTC;
    const int n0 = blockIdx.x * ROWS + mt * kSkinnyRows;
    const int K = a.K;
    // this warp's K range, in blocks of 32 (whole blocks; the ragged tail is zero-filled)
    const int blocks = (K + 31) >> 5;
    const int per = (blocks + KS - 1) / KS;
    const int b_lo = ks * per, b_hi = min(blocks, b_lo + per);
    const int r_lo = min(n0 + g, a.N - 1), r_hi = min(n0 + g + 8, a.N - 1);   // rows past N repeat the last one (never stored)
    const __half* w_lo = a.W + (size_t)r_lo * K + 8 * t;
    const __half* w_hi = a.W + (size_t)r_hi * K + 8 * t;
    const __half* xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) xrow[j] = a.X + (size_t)min(j * 8 + g, a.J - 1) * a.ldx + 8 * t;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 8
    for (int b = b_lo; b < b_hi; ++b) {
        const int k = b * 32 + 8 * t;          // first of this thread's 8 consecutive k
        const bool in = k < K;                 // K % 8 == 0: a thread's 8 positions are all inside or all outside
        const uint4 wl = in ? ldg_stream_v4(w_lo + (size_t)b * 32) : zero;
        const uint4 wh = in ? ldg_stream_v4(w_hi + (size_t)b * 32) : zero;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint4 xv = in ? __ldg(reinterpret_cast<const uint4*>(xrow[j] + (size_t)b * 32)) : zero;
            // two products per 32-wide block: k positions {0,1 | 2,3} and {4,5 | 6,7} of the thread's eight
            mma16816(acc[j], wl.x, wh.x, wl.y, wh.y, xv.x, xv.y);
            mma16816(acc[j], wl.z, wh.z, wl.w, wh.w, xv.z, xv.w);
        }
    }
    // accumulator layout: (row g, cols 2t, 2t+1), (row g+8, same cols) of each n-tile
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        part[ks][mt * 16 + g][j * 8 + 2 * t] = acc[j][0];
        part[ks][mt * 16 + g][j * 8 + 2 * t + 1] = acc[j][1];
        part[ks][mt * 16 + g + 8][j * 8 + 2 * t] = acc[j][2];
        part[ks][mt * 16 + g + 8][j * 8 + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    // output (activation row j, weight row r): consecutive threads take consecutive weight rows
    for (int i = threadIdx.x; i < ROWS * NT * 8; i += kSkinnyThreads) {
        const int r = i % ROWS, j = i / ROWS;
        const int n = blockIdx.x * ROWS + r;
        if (n >= a.N || j >= a.J) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < KS; ++w) v += part[w][r][j];
        if (a.bias) v += __half2float(a.bias[n]);
        if (a.act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
        if (a.y_is_f32) static_cast<float*>(a.Y)[(size_t)j * a.ldy + n] = v;
        else static_cast<__half*>(a.Y)[(size_t)j * a.ldy + n] = __float2half_rn(v);
    }
}
}  // namespace

// PIMB200_ERR_UNSUPPORTED when the shape is not this kernel's (the caller then takes the tensor-core or SIMT path)
int launch_gemm_wx_skinny(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                          int ldy, int act, int y_is_f32, cudaStream_t st) {
    if (J < 1 || J > kSkinnyMaxJ || K % 8 != 0 || ldx % 8 != 0 || !aligned16(W) || !aligned16(X)) return PIMB200_ERR_UNSUPPORTED;
    SkinnyArgs a{W, X, bias, Y, N, K, J, ldx, ldy, act, y_is_f32};
    const int nt = ceil_div(J, 8);
    if (N >= 2048) {
        const int grid = ceil_div(N, 2 * kSkinnyRows);
        switch (nt) {
            case 1: gemm_skinny_kernel<1, 2><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            case 2: gemm_skinny_kernel<2, 2><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            case 3: gemm_skinny_kernel<3, 2><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            default: gemm_skinny_kernel<4, 2><<<grid, kSkinnyThreads, 0, st>>>(a); break;
        }
    } else {
        const int grid = ceil_div(N, kSkinnyRows);
        switch (nt) {
            case 1: gemm_skinny_kernel<1, 1><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            case 2: gemm_skinny_kernel<2, 1><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            case 3: gemm_skinny_kernel<3, 1><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            default: gemm_skinny_kernel<4, 1><<<grid, kSkinnyThreads, 0, st>>>(a); break;
        }
    }
    return launch_status();
}

}  // namespace pimb200
