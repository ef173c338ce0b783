// Batched-stream linear layer for few activation rows:  Y[J, N] = act(X[J, K] . W[N, K]^T + bias[N]),  J <= 32.
//
// This is the batch 8 / 32 form of the batch-1 GEMV (several utterance streams sharing one weight matrix, or the
// branches of a MULTISTREAM node): the arithmetic intensity is J flop per weight byte, far below the ridge, so the
// bound is the one pass over W from HBM, exactly as for the GEMV.  A 128-row tcgen05 tile per CTA leaves most SMs
// without work at N = 4096 (32 CTAs) and costs a fixed pipeline set-up; here every SM streams W instead:
//   * a CTA owns 16 or 32 weight rows (one or two 16-row tiles) and its 8 warps split K between them; with 32 rows
//     (N >= 2048: one CTA per SM at N = 4096) a warp multiplies both tiles by the same X fragments; every load of a
//     group of K blocks is issued before the previous group's products, so 8 KB per warp are in flight;
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
constexpr int kSkinnyMaxBlockedJ = 256;                     // column-blocked form: at most 8 blocks of 32 rows ...
constexpr int kSkinnyMaxBlockedN = 2048;                    // ... of a matrix of at most 16 tcgen05 row tiles ...
constexpr size_t kSkinnyMaxBlockedNK = (size_t)8 << 20;     // ... and 16 MB

// not volatile: the compiler may move these loads and products freely (volatile asm statements keep their order, which
// would put every block's loads behind the previous block's products and serialise the HBM round trips)
__device__ __forceinline__ void mma16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_w(const __half* p) {
    uint4 r;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

struct SkinnyArgs {
    const __half* W;      // [N, K] row-major
    const __half* X;      // [J, ldx]
    const __half* bias;   // [N] or NULL
    void* Y;              // [J, ldy] fp16 or fp32
    int N, K, J, ldx, ldy, act, y_is_f32;
};

// NT: n-tiles of 8 activation rows; MTW: 16-row weight tiles per warp (1 or 2; they share the warp's X fragments).
// The 8 warps of a CTA split K; a warp walks its K range in groups of UB 32-wide blocks, the loads of the next group
// in flight while the current one is multiplied.
template <int NT, int MTW>
__global__ void __launch_bounds__(kSkinnyThreads) gemm_skinny_kernel(SkinnyArgs a) {
    constexpr int KS = kSkinnyWarps;
    constexpr int ROWS = MTW * kSkinnyRows;
    constexpr int UB = 4 / MTW;
    __shared__ float part[KS][ROWS][NT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    const int K = a.K;
    // this warp's K range, in blocks of 32 (whole blocks; the ragged tail is zero-filled)
    const int blocks = (K + 31) >> 5;
    const int per = (blocks + KS - 1) / KS;
    const int b_lo = warp * per, b_hi = min(blocks, b_lo + per);
    const __half* wrow[MTW][2];   // rows past N repeat the last one (never stored)
#pragma unroll
    for (int m = 0; m < MTW; ++m) {
        wrow[m][0] = a.W + (size_t)min(n0 + m * 16 + g, a.N - 1) * K + 8 * t;
        wrow[m][1] = a.W + (size_t)min(n0 + m * 16 + g + 8, a.N - 1) * K + 8 * t;
    }
    const __half* xrow[NT];
    const int j_base = blockIdx.y * kSkinnyMaxJ;               // this CTA's block of up to 32 activation rows
    const int j_rem = a.J - j_base;
#pragma unroll
    for (int j = 0; j < NT; ++j) xrow[j] = a.X + (size_t)(j_base + min(j * 8 + g, j_rem - 1)) * a.ldx + 8 * t;
    float acc[MTW][NT][4];
#pragma unroll
    for (int m = 0; m < MTW; ++m)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][j][i] = 0.f;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 wc[UB][MTW][2], xc[UB][NT], wn[UB][MTW][2], xn[UB][NT];
    auto load_group = [&](uint4 (&w)[UB][MTW][2], uint4 (&x)[UB][NT], int b0) {
#pragma unroll
        for (int u = 0; u < UB; ++u) {
            const int b = b0 + u;
            // K % 8 == 0: a thread's 8 consecutive k are all inside or all outside
            const bool in = b < b_hi && b * 32 + 8 * t < K;
#pragma unroll
            for (int m = 0; m < MTW; ++m) {
                w[u][m][0] = in ? ldg_w(wrow[m][0] + (size_t)b * 32) : zero;
                w[u][m][1] = in ? ldg_w(wrow[m][1] + (size_t)b * 32) : zero;
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) x[u][j] = in ? __ldg(reinterpret_cast<const uint4*>(xrow[j] + (size_t)b * 32)) : zero;
        }
    };
    auto multiply = [&](const uint4 (&w)[UB][MTW][2], const uint4 (&x)[UB][NT]) {
#pragma unroll
        for (int u = 0; u < UB; ++u)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int m = 0; m < MTW; ++m) {
                    // two products per 32-wide block: k positions {0,1 | 2,3} and {4,5 | 6,7} of the thread's eight
                    mma16816(acc[m][j], w[u][m][0].x, w[u][m][1].x, w[u][m][0].y, w[u][m][1].y, x[u][j].x, x[u][j].y);
                    mma16816(acc[m][j], w[u][m][0].z, w[u][m][1].z, w[u][m][0].w, w[u][m][1].w, x[u][j].z, x[u][j].w);
                }
    };
    // two register buffers used alternately (no copies between them: a move would wait for the load it moves)
    load_group(wc, xc, b_lo);
    for (int b0 = b_lo; b0 < b_hi; b0 += 2 * UB) {
        load_group(wn, xn, b0 + UB);
        multiply(wc, xc);
        load_group(wc, xc, b0 + 2 * UB);
        multiply(wn, xn);
    }
    // accumulator layout: (row g, cols 2t, 2t+1), (row g+8, same cols) of each n-tile
#pragma unroll
    for (int m = 0; m < MTW; ++m)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            part[warp][m * 16 + g][j * 8 + 2 * t] = acc[m][j][0];
            part[warp][m * 16 + g][j * 8 + 2 * t + 1] = acc[m][j][1];
            part[warp][m * 16 + g + 8][j * 8 + 2 * t] = acc[m][j][2];
            part[warp][m * 16 + g + 8][j * 8 + 2 * t + 1] = acc[m][j][3];
        }
    __syncthreads();
    // output (activation row j, weight row r): consecutive threads take consecutive weight rows
    for (int i = threadIdx.x; i < ROWS * NT * 8; i += kSkinnyThreads) {
        const int r = i % ROWS, j = i / ROWS;
        const int n = n0 + r;
        if (n >= a.N || j >= j_rem) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < KS; ++w) v += part[w][r][j];
        if (a.bias) v += __half2float(a.bias[n]);
        if (a.act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
        if (a.y_is_f32) static_cast<float*>(a.Y)[(size_t)(j_base + j) * a.ldy + n] = v;
        else static_cast<__half*>(a.Y)[(size_t)(j_base + j) * a.ldy + n] = __float2half_rn(v);
    }
}

// Many weight rows (N >= 16384: the vocabulary projection of a batched decode step) and 9..32 activation rows: one
// warp per 16-row tile over the whole of K, no K split, so nothing is folded through shared memory and no barrier
// follows the start.  Read straight from global memory the X fragments would cost as many load slots and registers as
// W itself; here the CTA copies X into shared memory once (cp.async; odd rows stored with their 16-byte chunks swapped
// across 64 bytes, so a quarter-warp's 128-bit reads - two rows x 64 bytes - fall in distinct banks) and its 8 warps
// walk tiles of a persistent grid, two register buffers of W loads in flight per warp.
// Several independent products in ONE launch (the branches of a MULTISTREAM node: a few activation rows against
// different weight matrices): blockIdx.z selects the problem, blockIdx.y its block of 32 activation rows, blockIdx.x its
// 16-row weight tile; CTAs past a problem's extent leave at once.  Same arithmetic as gemm_skinny_kernel<NT, 1>.
constexpr int kGroupedMax = 8;
struct GroupedArgs {
    SkinnyArgs p[kGroupedMax];
};

template <int NT>
__global__ void __launch_bounds__(kSkinnyThreads) gemm_skinny_grouped_kernel(const __grid_constant__ GroupedArgs ga) {
    constexpr int KS = kSkinnyWarps;
    constexpr int UB = 4;
    __shared__ float part[KS][kSkinnyRows][NT * 8 + 1];
    const SkinnyArgs& a = ga.p[blockIdx.z];
    const int n0 = blockIdx.x * kSkinnyRows;
    const int j_base = blockIdx.y * kSkinnyMaxJ;
    if (n0 >= a.N || j_base >= a.J) return;                    // CTA-uniform
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int K = a.K;
    const int blocks = (K + 31) >> 5;
    const int per = (blocks + KS - 1) / KS;
    const int b_lo = warp * per, b_hi = min(blocks, b_lo + per);
    const __half* w_lo = a.W + (size_t)min(n0 + g, a.N - 1) * K + 8 * t;
    const __half* w_hi = a.W + (size_t)min(n0 + g + 8, a.N - 1) * K + 8 * t;
    const int j_rem = a.J - j_base;
    const __half* xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) xrow[j] = a.X + (size_t)(j_base + min(j * 8 + g, j_rem - 1)) * a.ldx + 8 * t;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    uint4 wc[UB][2], xc[UB][NT], wn[UB][2], xn[UB][NT];
    auto load_group = [&](uint4 (&w)[UB][2], uint4 (&x)[UB][NT], int b0) {
#pragma unroll
        for (int u = 0; u < UB; ++u) {
            const int b = b0 + u;
            const bool in = b < b_hi && b * 32 + 8 * t < K;
            w[u][0] = in ? ldg_w(w_lo + (size_t)b * 32) : zero;
            w[u][1] = in ? ldg_w(w_hi + (size_t)b * 32) : zero;
#pragma unroll
            for (int j = 0; j < NT; ++j) x[u][j] = in ? __ldg(reinterpret_cast<const uint4*>(xrow[j] + (size_t)b * 32)) : zero;
        }
    };
    auto multiply = [&](const uint4 (&w)[UB][2], const uint4 (&x)[UB][NT]) {
#pragma unroll
        for (int u = 0; u < UB; ++u)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                mma16816(acc[j], w[u][0].x, w[u][1].x, w[u][0].y, w[u][1].y, x[u][j].x, x[u][j].y);
                mma16816(acc[j], w[u][0].z, w[u][1].z, w[u][0].w, w[u][1].w, x[u][j].z, x[u][j].w);
            }
    };
    load_group(wc, xc, b_lo);
    for (int b0 = b_lo; b0 < b_hi; b0 += 2 * UB) {
        load_group(wn, xn, b0 + UB);
        multiply(wc, xc);
        load_group(wc, xc, b0 + 2 * UB);
        multiply(wn, xn);
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        part[warp][g][j * 8 + 2 * t] = acc[j][0];
        part[warp][g][j * 8 + 2 * t + 1] = acc[j][1];
        part[warp][g + 8][j * 8 + 2 * t] = acc[j][2];
        part[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kSkinnyRows * NT * 8; i += kSkinnyThreads) {
        const int r = i % kSkinnyRows, j = i / kSkinnyRows;
        const int n = n0 + r;
        if (n >= a.N || j >= j_rem) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < KS; ++w) v += part[w][r][j];
        if (a.bias) v += __half2float(a.bias[n]);
        if (a.act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
        if (a.y_is_f32) static_cast<float*>(a.Y)[(size_t)(j_base + j) * a.ldy + n] = v;
        else static_cast<__half*>(a.Y)[(size_t)(j_base + j) * a.ldy + n] = __float2half_rn(v);
    }
}

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 r;
    asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}

template <int NT, bool FULL>   // FULL: K a multiple of 128 (no partial group of K blocks)
__global__ void __launch_bounds__(kSkinnyThreads, 2) gemm_skinny_rows_kernel(SkinnyArgs a, int tiles) {
    constexpr int UB = 4;                                            // 32-wide K blocks per register buffer
    extern __shared__ __align__(16) unsigned char sk_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int K = a.K;                                               // K % 64 == 0 (checked by the launcher)
    const int xs = K * 2;                                            // bytes per X row, a multiple of 128
    const int blocks = K >> 5;
    const int gpt = (blocks + UB - 1) / UB;                          // groups of K blocks per tile
    {
        const int chunks = K >> 3;                                   // 16-byte chunks per row
        for (int row = warp; row < NT * 8; row += kSkinnyWarps) {
            const __half* src = a.X + (size_t)min(row, a.J - 1) * a.ldx;   // rows past J repeat the last one
            unsigned char* dst = sk_smem + (size_t)row * xs;
            const int flip = (row & 1) << 2;
            for (int c = lane; c < chunks; c += 32)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst + ((c ^ flip) << 4))),
                             "l"(src + c * 8) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // tile i of the launch belongs to CTA i % gridDim.x, warp (i / gridDim.x) % 8; a warp walks its tiles as one stream of
    // (tile, group) pairs, so the loads of a tile's first group are in flight during the previous tile's last products
    const int stride = kSkinnyWarps * gridDim.x;
    uint4 w0[UB][2], w1[UB][2];
    auto load_group = [&](uint4 (&w)[UB][2], int tile, int grp) {
        if (tile >= tiles) return;                                   // warp-uniform
        const int n0 = tile * kSkinnyRows;
        const __half* p_lo = a.W + (size_t)min(n0 + g, a.N - 1) * K + 8 * t + grp * (UB * 32);   // rows past N repeat the last
        const __half* p_hi = a.W + (size_t)min(n0 + g + 8, a.N - 1) * K + 8 * t + grp * (UB * 32);
#pragma unroll
        for (int u = 0; u < UB; ++u)
            if (FULL || grp * UB + u < blocks) {
                w[u][0] = ldg_w(p_lo + u * 32);
                w[u][1] = ldg_w(p_hi + u * 32);
            }
    };
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const uint32_t xaddr = (uint32_t)__cvta_generic_to_shared(sk_smem) + (uint32_t)(g * xs + t * 16);
    const int s1 = g & 1;                                            // odd rows: 64-byte halves of a 128-byte pair swapped
    auto step = [&](const uint4 (&w)[UB][2], int tile, int grp) {
#pragma unroll
        for (int u = 0; u < UB; ++u)
            if (FULL || grp * UB + u < blocks) {
                const uint32_t xb = xaddr + (uint32_t)(((grp * UB + u) ^ s1) << 6);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const uint4 xv = lds_v4(xb + (uint32_t)(j * 8 * xs));
                    mma16816(acc[j], w[u][0].x, w[u][1].x, w[u][0].y, w[u][1].y, xv.x, xv.y);
                    mma16816(acc[j], w[u][0].z, w[u][1].z, w[u][0].w, w[u][1].w, xv.z, xv.w);
                }
            }
        if (grp != gpt - 1) return;
        // the tile is complete.  Accumulator layout: (row g, cols 2t, 2t+1), (row g+8, same cols) of each n-tile
        const int n0 = tile * kSkinnyRows;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int n = n0 + g + 8 * h;
            const float bv = (a.bias && n < a.N) ? __half2float(a.bias[n]) : 0.f;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int col = j * 8 + 2 * t + e;
                    float v = acc[j][2 * h + e] + bv;
                    acc[j][2 * h + e] = 0.f;
                    if (n >= a.N || col >= a.J) continue;
                    if (a.act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
                    if (a.y_is_f32) static_cast<float*>(a.Y)[(size_t)col * a.ldy + n] = v;
                    else static_cast<__half*>(a.Y)[(size_t)col * a.ldy + n] = __float2half_rn(v);
                }
        }
    };
    auto advance = [&](int& tile, int& grp) {
        if (++grp == gpt) { grp = 0; tile += stride; }
    };
    int lt = blockIdx.x + warp * gridDim.x, lg = 0;                  // load cursor
    int ct = lt, cg = 0;                                             // compute cursor
    load_group(w0, lt, lg); advance(lt, lg);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                                 // reached by every warp, with or without a tile
    while (ct < tiles) {
        load_group(w1, lt, lg); advance(lt, lg);
        step(w0, ct, cg); advance(ct, cg);
        if (ct >= tiles) break;
        load_group(w0, lt, lg); advance(lt, lg);
        step(w1, ct, cg); advance(ct, cg);
    }
}

template <int NT>
int launch_skinny_rows(const SkinnyArgs& a, cudaStream_t st) {
    const size_t smem = (size_t)NT * 8 * a.K * 2;
    if (a.K % 64 != 0 || smem > 200 * 1024) return PIMB200_ERR_UNSUPPORTED;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return PIMB200_ERR_UNSUPPORTED;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(gemm_skinny_rows_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_skinny_rows_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return PIMB200_ERR_LAUNCH;
        attr_set[dev] = true;
    }
    const int tiles = ceil_div(a.N, kSkinnyRows);
    const int per_sm = smem <= 110 * 1024 ? 2 : 1;
    DeviceCtx* ctx = current_ctx();
    const int grid = min(ceil_div(tiles, kSkinnyWarps), (ctx ? ctx->sm_count : kNumSmB200) * per_sm);
    if (a.K % 128 == 0) gemm_skinny_rows_kernel<NT, true><<<grid, kSkinnyThreads, smem, st>>>(a, tiles);
    else gemm_skinny_rows_kernel<NT, false><<<grid, kSkinnyThreads, smem, st>>>(a, tiles);
    return launch_status();
}
}  // namespace

// PIMB200_ERR_UNSUPPORTED when the shape is not this kernel's (the caller then takes the tensor-core or SIMT path)
int launch_gemm_wx_skinny(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                          int ldy, int act, int y_is_f32, cudaStream_t st) {
    if (J < 1 || K % 8 != 0 || ldx % 8 != 0 || !aligned16(W) || !aligned16(X)) return PIMB200_ERR_UNSUPPORTED;
    // More than 32 activation rows run as column blocks of 32 (grid.y) when the weight matrix is small: W then comes
    // from L2 for all but the first block, and a matrix of a few 128-row tiles would leave most SMs of the tcgen05
    // kernel's grid without work (a Transformer layer's 512 x 512 projections for 128 sequences: 4 tiles).
    if (J > kSkinnyMaxJ && (J > kSkinnyMaxBlockedJ || N > kSkinnyMaxBlockedN || (size_t)N * K > kSkinnyMaxBlockedNK))
        return PIMB200_ERR_UNSUPPORTED;
    SkinnyArgs a{W, X, bias, Y, N, K, J, ldx, ldy, act, y_is_f32};
    const int nt = J > kSkinnyMaxJ ? 4 : ceil_div(J, 8);
    const int jblocks = ceil_div(J, kSkinnyMaxJ);
    if (nt >= 2 && N >= 16384 && jblocks == 1) {
        // a warp per row tile with X in shared memory, when the CTA's copy of X fits
        const int rc = nt == 2 ? launch_skinny_rows<2>(a, st) : nt == 3 ? launch_skinny_rows<3>(a, st) : launch_skinny_rows<4>(a, st);
        if (rc != PIMB200_ERR_UNSUPPORTED) return rc;
    }
    if (N >= 2048) {
        const dim3 grid(ceil_div(N, 2 * kSkinnyRows), jblocks);
        switch (nt) {
            case 1: gemm_skinny_kernel<1, 2><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            case 2: gemm_skinny_kernel<2, 2><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            case 3: gemm_skinny_kernel<3, 2><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            default: gemm_skinny_kernel<4, 2><<<grid, kSkinnyThreads, 0, st>>>(a); break;
        }
    } else {
        const dim3 grid(ceil_div(N, kSkinnyRows), jblocks);
        switch (nt) {
            case 1: gemm_skinny_kernel<1, 1><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            case 2: gemm_skinny_kernel<2, 1><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            case 3: gemm_skinny_kernel<3, 1><<<grid, kSkinnyThreads, 0, st>>>(a); break;
            default: gemm_skinny_kernel<4, 1><<<grid, kSkinnyThreads, 0, st>>>(a); break;
        }
    }
    return launch_status();
}

// Up to 8 problems in one launch; PIMB200_ERR_UNSUPPORTED when one of them is not a shape of the few-row kernels (the
// caller then launches them one by one)
int launch_gemm_wx_grouped(const GemmProblem* pr, int n, cudaStream_t st) {
    if (n < 1 || n > kGroupedMax) return PIMB200_ERR_UNSUPPORTED;
    GroupedArgs ga;
    int max_tiles = 0, max_jb = 0, max_j = 0;
    for (int i = 0; i < n; ++i) {
        const GemmProblem& q = pr[i];
        if (q.J < 1 || q.J > kSkinnyMaxBlockedJ || q.K % 8 != 0 || q.ldx % 8 != 0 || !aligned16(q.W) || !aligned16(q.X))
            return PIMB200_ERR_UNSUPPORTED;
        if (q.J > kSkinnyMaxJ && (q.N > kSkinnyMaxBlockedN || (size_t)q.N * q.K > kSkinnyMaxBlockedNK)) return PIMB200_ERR_UNSUPPORTED;
        ga.p[i] = SkinnyArgs{q.W, q.X, q.bias, q.Y, q.N, q.K, q.J, q.ldx, q.ldy, q.act, q.y_is_f32};
        max_tiles = max(max_tiles, ceil_div(q.N, kSkinnyRows));
        max_jb = max(max_jb, ceil_div(q.J, kSkinnyMaxJ));
        max_j = max(max_j, min(q.J, kSkinnyMaxJ));
    }
    for (int i = n; i < kGroupedMax; ++i) ga.p[i] = SkinnyArgs{nullptr, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, 0, 0};
    const dim3 grid(max_tiles, max_jb, n);
    switch (ceil_div(max_j, 8)) {
        case 1: gemm_skinny_grouped_kernel<1><<<grid, kSkinnyThreads, 0, st>>>(ga); break;
        case 2: gemm_skinny_grouped_kernel<2><<<grid, kSkinnyThreads, 0, st>>>(ga); break;
        case 3: gemm_skinny_grouped_kernel<3><<<grid, kSkinnyThreads, 0, st>>>(ga); break;
        default: gemm_skinny_grouped_kernel<4><<<grid, kSkinnyThreads, 0, st>>>(ga); break;
    }
    return launch_status();
}

}  // namespace pimb200
