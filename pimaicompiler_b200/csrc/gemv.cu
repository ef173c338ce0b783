// Batch-1 GEMV family, the SIMT GEMM fall-back and the fp16 glue ops.
//
// These kernels stand where the reference offloads to PIM-HBM (PimExecuteGemm) or launches its
// HIP GEMV templates (runtime/include/executor/op_executor/custom_ops.h).  All of them are
// HBM-bandwidth bound: 128-bit coalesced loads that bypass L1, fp32 accumulation, warp-shuffle
// reductions and the bias / ReLU epilogue fused into the same kernel.
#include <mutex>

#include "common.cuh"

namespace pimb200 {

// =============================================================================================
// MV:  y[n] = act(sum_k W[n,k] x[k] + b[n])
// One warp owns R consecutive rows; a lane walks the row in 16-byte chunks (stride 32 chunks),
// so a warp reads 512 contiguous bytes per row per iteration.  W bypasses L1 (read once); x is
// read through L1 (it is a few KB and every warp reads all of it) — staging it in shared memory
// first costs a barrier before the first weight load and measured slower.  R*unroll independent
// 16-byte loads are in flight per lane.
// =============================================================================================
template <int R>
__global__ void __launch_bounds__(256) gemv_mv_vec_kernel(const __half* __restrict__ W, const __half* __restrict__ x,
                                                          const __half* __restrict__ bias, __half* __restrict__ y,
                                                          int N, int K, int act) {
    const int K8 = K >> 3;
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = (blockIdx.x * (blockDim.x >> 5) + warp) * R;
    if (row0 >= N) return;

    const uint4* wrow[R];
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int row = min(row0 + r, N - 1);  // clamp: rows past N re-read the last row, never stored
        wrow[r] = reinterpret_cast<const uint4*>(W + (size_t)row * K);
        acc[r] = 0.f;
    }
#pragma unroll 4
    for (int c = lane; c < K8; c += 32) {
        float xf[8];
        widen8(__ldg(x4 + c), xf);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = dot8f(ldg_stream_v4(wrow[r] + c), xf, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int row = row0 + r;
            if (row < N) {
                float v = acc[r] + (bias ? __half2float(bias[row]) : 0.f);
                if (act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
                y[row] = __float2half_rn(v);
            }
        }
    }
}

// any K, any alignment: one warp per row, scalar half loads
__global__ void __launch_bounds__(256) gemv_mv_generic_kernel(const __half* __restrict__ W, const __half* __restrict__ x,
                                                              const __half* __restrict__ bias, __half* __restrict__ y,
                                                              int N, int K, int act) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= N) return;
    const __half* w = W + (size_t)row * K;
    float acc = 0.f;
    for (int k = lane; k < K; k += 32) acc = fmaf(__half2float(w[k]), __half2float(x[k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) {
        float v = acc + (bias ? __half2float(bias[row]) : 0.f);
        if (act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
        y[row] = __float2half_rn(v);
    }
}

static int launch_gemv_mv(const __half* W, const __half* x, const __half* bias, __half* y, int N, int K, int act,
                          cudaStream_t st) {
    const bool vec = (K % 8 == 0) && aligned16(W) && aligned16(x);
    if (!vec) {
        gemv_mv_generic_kernel<<<ceil_div(N, 8), 256, 0, st>>>(W, x, bias, y, N, K, act);
        return launch_status();
    }
    // rows per warp: enough warps to cover every SM several times, else fewer rows per warp
    const long warps4 = ((long)N + 3) / 4, warps2 = ((long)N + 1) / 2;
    const long want = (long)kNumSmB200 * 8 * 2;
    const int R = warps4 >= want ? 4 : (warps2 >= want ? 2 : 1);
    const int grid = ceil_div(N, 8 * R);
    if (R == 4) gemv_mv_vec_kernel<4><<<grid, 256, 0, st>>>(W, x, bias, y, N, K, act);
    else if (R == 2) gemv_mv_vec_kernel<2><<<grid, 256, 0, st>>>(W, x, bias, y, N, K, act);
    else gemv_mv_vec_kernel<1><<<grid, 256, 0, st>>>(W, x, bias, y, N, K, act);
    return launch_status();
}

// =============================================================================================
// VM:  y[n] = act(sum_k x[k] A[k,n] + b[n]),  A row-major [K,N]
// Threads run along n (8 columns = one 16-byte load each), so every row segment a warp touches
// is contiguous.  LPR lanes cover one row segment (LPR*8 columns); a warp covers 32/LPR rows
// per pass and the CTA's 8 warps cover 8*32/LPR rows.  K is additionally split over gridDim.y
// CTAs; their fp32 partial sums go through the per-device scratch and the CTA that draws the
// last ticket for a column tile reduces them and applies the epilogue.
// =============================================================================================
template <int LPR>
__global__ void __launch_bounds__(256) gemv_vm_vec_kernel(const __half* __restrict__ x, const __half* __restrict__ A,
                                                          const __half* __restrict__ bias, __half* __restrict__ y,
                                                          int K, int N, int act, int rows_per_split,
                                                          float* __restrict__ partials,
                                                          unsigned int* __restrict__ tickets) {
    constexpr int TILE = LPR * 8;        // columns per CTA
    constexpr int RPW = 32 / LPR;        // rows per warp per pass
    __shared__ float red[8][TILE];
    __shared__ int s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR, cl = lane % LPR;
    const int col = blockIdx.x * TILE + cl * 8;
    const int S = gridDim.y, split = blockIdx.y;
    const int k0 = split * rows_per_split;
    const int k1 = min(K, k0 + rows_per_split);

    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (col < N) {
#pragma unroll 8
        for (int k = k0 + warp * RPW + sub; k < k1; k += 8 * RPW) {
            const uint4 a = ldg_stream_v4(A + (size_t)k * N + col);
            const float xk = __half2float(__ldg(x + k));
            float2 f;
            f = h2f2(a.x); acc[0] = fmaf(xk, f.x, acc[0]); acc[1] = fmaf(xk, f.y, acc[1]);
            f = h2f2(a.y); acc[2] = fmaf(xk, f.x, acc[2]); acc[3] = fmaf(xk, f.y, acc[3]);
            f = h2f2(a.z); acc[4] = fmaf(xk, f.x, acc[4]); acc[5] = fmaf(xk, f.y, acc[5]);
            f = h2f2(a.w); acc[6] = fmaf(xk, f.x, acc[6]); acc[7] = fmaf(xk, f.y, acc[7]);
        }
    }
    // fold the row groups of a warp together, then the warps through shared memory
#pragma unroll
    for (int o = 16; o >= LPR; o >>= 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    }
    if (sub == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) red[warp][cl * 8 + j] = acc[j];
    }
    __syncthreads();
    const int t = threadIdx.x;
    const int ocol = blockIdx.x * TILE + t;
    float v = 0.f;
    if (t < TILE) {
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][t];
    }
    if (S > 1) {
        if (t < TILE && ocol < N) __stcg(partials + (size_t)split * N + ocol, v);
        __threadfence();
        __syncthreads();
        if (t == 0) {
            unsigned int tk = atomicAdd(tickets + blockIdx.x, 1u);
            s_last = (tk == (unsigned)(S - 1));
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        v = 0.f;
        if (t < TILE && ocol < N) {
            for (int s = 0; s < S; ++s) v += __ldcg(partials + (size_t)s * N + ocol);
        }
        if (t == 0) tickets[blockIdx.x] = 0;  // leave the ticket counter clean for the next call
    }
    if (t < TILE && ocol < N) {
        v += bias ? __half2float(bias[ocol]) : 0.f;
        if (act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
        y[ocol] = __float2half_rn(v);
    }
}

// any N, any alignment: one thread per column, rows split across the 8 warps of a CTA
__global__ void __launch_bounds__(256) gemv_vm_generic_kernel(const __half* __restrict__ x, const __half* __restrict__ A,
                                                              const __half* __restrict__ bias, __half* __restrict__ y,
                                                              int K, int N, int act) {
    __shared__ float red[8][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * 32 + lane;
    float acc = 0.f;
    if (col < N)
        for (int k = warp; k < K; k += 8) acc = fmaf(__half2float(x[k]), __half2float(A[(size_t)k * N + col]), acc);
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < N) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][lane];
        v += bias ? __half2float(bias[col]) : 0.f;
        if (act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
        y[col] = __float2half_rn(v);
    }
}

// Chooses the column-tile width and the K split.  Exposed so the scratch-free entry point can
// reuse the same plan with its own scratch.
struct VmPlan {
    int lpr;             // lanes per row segment: 32 or 8
    int tiles;           // gridDim.x
    int splits;          // gridDim.y
    int rows_per_split;
};
VmPlan plan_gemv_vm(int K, int N, size_t max_partial_floats, int max_tiles) {
    VmPlan p;
    p.lpr = (ceil_div(N, 256) >= kNumSmB200 / 4) ? 32 : 8;
    const int tile = p.lpr * 8;
    p.tiles = ceil_div(N, tile);
    const int rows_per_pass = 8 * (32 / p.lpr);       // rows a CTA covers per pass
    int want = ceil_div(4 * kNumSmB200, p.tiles);     // about four CTAs per SM
    int max_by_rows = K / (rows_per_pass * 4);        // keep at least four passes per CTA
    if (max_by_rows < 1) max_by_rows = 1;
    int S = want < max_by_rows ? want : max_by_rows;
    if (S < 1) S = 1;
    if (p.tiles > max_tiles) S = 1;
    while (S > 1 && (size_t)S * (size_t)N > max_partial_floats) --S;
    p.rows_per_split = ceil_div(K, S);
    p.splits = ceil_div(K, p.rows_per_split);
    return p;
}

int launch_gemv_vm_with_scratch(const __half* x, const __half* A, const __half* bias, __half* y, int K, int N,
                                int act, const VmPlan& p, float* partials, unsigned int* tickets, cudaStream_t st) {
    dim3 grid(p.tiles, p.splits);
    if (p.lpr == 32)
        gemv_vm_vec_kernel<32><<<grid, 256, 0, st>>>(x, A, bias, y, K, N, act, p.rows_per_split, partials, tickets);
    else
        gemv_vm_vec_kernel<8><<<grid, 256, 0, st>>>(x, A, bias, y, K, N, act, p.rows_per_split, partials, tickets);
    return launch_status();
}

static std::mutex g_vm_mutex;
static cudaStream_t g_vm_last_stream[64];
static bool g_vm_used[64];
static cudaEvent_t g_vm_event[64];   // recorded behind the last split-K user of the device's scratch

// Calls on one device share the split-K scratch.  Every split-K launch records an event behind itself on its own
// stream (scratch_user_done); a later caller on a different stream waits for that event first.  Nothing is ever
// recorded on a stream handle remembered from an earlier call (the caller may have destroyed it since).
// While a stream is being captured into a CUDA graph neither side is possible: captured launches are not ordered
// against other users of the scratch, so replays of graphs that contain split-K VM products must be ordered by
// the caller against every other VM call on the device.
static int order_scratch_users(int dev, cudaStream_t st) {
    if (dev < 0 || dev >= 64) return PIMB200_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(g_vm_mutex);
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(st, &cs);
    if (cs != cudaStreamCaptureStatusNone) return PIMB200_OK;
    if (g_vm_used[dev] && g_vm_last_stream[dev] != st) PIMB200_CUDA_TRY(cudaStreamWaitEvent(st, g_vm_event[dev], 0));
    return PIMB200_OK;
}
static int scratch_user_done(int dev, cudaStream_t st) {
    if (dev < 0 || dev >= 64) return PIMB200_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(g_vm_mutex);
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(st, &cs);
    if (cs != cudaStreamCaptureStatusNone) return PIMB200_OK;
    if (!g_vm_event[dev]) PIMB200_CUDA_TRY(cudaEventCreateWithFlags(&g_vm_event[dev], cudaEventDisableTiming));
    PIMB200_CUDA_TRY(cudaEventRecord(g_vm_event[dev], st));
    g_vm_used[dev] = true;
    g_vm_last_stream[dev] = st;
    return PIMB200_OK;
}

static int launch_gemv_vm(const __half* x, const __half* A, const __half* bias, __half* y, int K, int N, int act,
                          bool allow_split, cudaStream_t st) {
    const bool vec = (N % 8 == 0) && aligned16(A);
    if (!vec) {
        gemv_vm_generic_kernel<<<ceil_div(N, 32), 256, 0, st>>>(x, A, bias, y, K, N, act);
        return launch_status();
    }
    float* partials = nullptr;
    unsigned int* tickets = nullptr;
    VmPlan p;
    int dev = -1;
    if (allow_split) {
        DeviceCtx* ctx = current_ctx();
        if (!ctx) return PIMB200_ERR_NOT_INIT;
        p = plan_gemv_vm(K, N, kSplitKMaxFloats, kSplitKMaxTiles);
        if (p.splits > 1) {
            PIMB200_CUDA_TRY(cudaGetDevice(&dev));
            int rc = order_scratch_users(dev, st);
            if (rc != PIMB200_OK) return rc;
            partials = ctx->splitk_partials;
            tickets = ctx->splitk_tickets;
        }
    } else {
        p = plan_gemv_vm(K, N, 0, 0);  // forces a single split
    }
    const int rc = launch_gemv_vm_with_scratch(x, A, bias, y, K, N, act, p, partials, tickets, st);
    if (rc == PIMB200_OK && dev >= 0) return scratch_user_done(dev, st);
    return rc;
}

// =============================================================================================
// VV dot product: one CTA, fp32 accumulate
// =============================================================================================
__global__ void __launch_bounds__(256) dot_vv_kernel(const __half* __restrict__ a, const __half* __restrict__ b,
                                                     __half* __restrict__ y, int K) {
    __shared__ float red[8];
    float acc = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) acc = fmaf(__half2float(a[k]), __half2float(b[k]), acc);
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w];
        y[0] = __float2half_rn(v);
    }
}

// =============================================================================================
// fp16 add, same-shape or row-broadcast, any n
// =============================================================================================
__global__ void __launch_bounds__(256) add_f16_vec_kernel(const uint4* A, const uint4* __restrict__ B,
                                                          uint4* C, size_t total8, int n8, int bcast) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        uint4 a = A[i];
        uint4 b = B[bcast ? (i % n8) : i];
        uint4 c;
        __half2* ap = reinterpret_cast<__half2*>(&a);
        __half2* bp = reinterpret_cast<__half2*>(&b);
        __half2* cp = reinterpret_cast<__half2*>(&c);
#pragma unroll
        for (int j = 0; j < 4; ++j) cp[j] = __hadd2(ap[j], bp[j]);
        C[i] = c;
    }
}
__global__ void __launch_bounds__(256) add_f16_scalar_kernel(const __half* A, const __half* __restrict__ B,
                                                             __half* C, size_t total, int n, int bcast) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        C[i] = __hadd(A[i], B[bcast ? (i % n) : i]);
}

// =============================================================================================
// strided copies (copy_ into a slice, cat along the inner dimension)
// =============================================================================================
template <typename V>
__global__ void __launch_bounds__(256) copy_2d_kernel(unsigned char* __restrict__ dst, size_t dpitch,
                                                      const unsigned char* __restrict__ src, size_t spitch,
                                                      size_t row_elems, size_t rows) {
    const size_t total = row_elems * rows;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i / row_elems, c = i - r * row_elems;
        *reinterpret_cast<V*>(dst + r * dpitch + c * sizeof(V)) =
            *reinterpret_cast<const V*>(src + r * spitch + c * sizeof(V));
    }
}

static int launch_copy_2d(void* dst, size_t dpitch, const void* src, size_t spitch, size_t row_bytes, size_t rows,
                          cudaStream_t st) {
    if (row_bytes == 0 || rows == 0) return PIMB200_OK;
    if (dpitch == row_bytes && spitch == row_bytes) {
        PIMB200_CUDA_TRY(cudaMemcpyAsync(dst, src, row_bytes * rows, cudaMemcpyDeviceToDevice, st));
        return PIMB200_OK;
    }
    unsigned char* d = static_cast<unsigned char*>(dst);
    const unsigned char* s = static_cast<const unsigned char*>(src);
    const uintptr_t bits = reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(s) | dpitch | spitch | row_bytes;
    const size_t total_bytes = row_bytes * rows;
    auto grid_for = [](size_t elems) {
        size_t g = (elems + 255) / 256;
        return (unsigned)(g > 148 * 16 ? 148 * 16 : (g ? g : 1));
    };
    if ((bits & 15) == 0)
        copy_2d_kernel<uint4><<<grid_for(total_bytes / 16), 256, 0, st>>>(d, dpitch, s, spitch, row_bytes / 16, rows);
    else if ((bits & 3) == 0)
        copy_2d_kernel<uint32_t><<<grid_for(total_bytes / 4), 256, 0, st>>>(d, dpitch, s, spitch, row_bytes / 4, rows);
    else if ((bits & 1) == 0)
        copy_2d_kernel<uint16_t><<<grid_for(total_bytes / 2), 256, 0, st>>>(d, dpitch, s, spitch, row_bytes / 2, rows);
    else
        copy_2d_kernel<uint8_t><<<grid_for(total_bytes), 256, 0, st>>>(d, dpitch, s, spitch, row_bytes, rows);
    return launch_status();
}

// =============================================================================================
// SIMT GEMM fall-back:  Y[j,n] = act(sum_k X[j,k] W[n,k] + b[n]) — any shape, any alignment.
// 64x64 output tile, 32-deep k slab, 256 threads with a 4x4 register tile each.
// The tensor-core kernel in gemm_tc.cu takes the shapes it supports; this one takes the rest.
// =============================================================================================
template <bool OUT_F32>
__global__ void __launch_bounds__(256) gemm_wx_simt_kernel(const __half* __restrict__ W, const __half* __restrict__ X,
                                                           const __half* __restrict__ bias, void* __restrict__ Yv,
                                                           int N, int K, int J, int ldx, int ldy, int act) {
    constexpr int BN = 64, BJ = 64, BK = 32;
    __shared__ __align__(16) float Ws[BK][BN + 4];
    __shared__ __align__(16) float Xs[BK][BJ + 4];
    const int n0 = blockIdx.x * BN, j0 = blockIdx.y * BJ;
    const int tn = threadIdx.x & 15, tj = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;

    const int lrow = threadIdx.x >> 2;        // 0..63: tile row this thread loads
    const int lk = (threadIdx.x & 3) * 8;     // 0,8,16,24: first k of its 8-wide slice
    for (int kb = 0; kb < K; kb += BK) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int k = kb + lk + e;
            const int n = n0 + lrow, j = j0 + lrow;
            Ws[lk + e][lrow] = (n < N && k < K) ? __half2float(W[(size_t)n * K + k]) : 0.f;
            Xs[lk + e][lrow] = (j < J && k < K) ? __half2float(X[(size_t)j * ldx + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 wv = *reinterpret_cast<const float4*>(&Ws[kk][tn * 4]);
            const float4 xv = *reinterpret_cast<const float4*>(&Xs[kk][tj * 4]);
            const float w4[4] = {wv.x, wv.y, wv.z, wv.w};
            const float x4[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(x4[a], w4[b], acc[a][b]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int j = j0 + tj * 4 + a;
        if (j >= J) continue;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int n = n0 + tn * 4 + b;
            if (n >= N) continue;
            float v = acc[a][b] + (bias ? __half2float(bias[n]) : 0.f);
            if (act == PIMB200_ACT_RELU) v = fmaxf(v, 0.f);
            if (OUT_F32)
                static_cast<float*>(Yv)[(size_t)j * ldy + n] = v;
            else
                static_cast<__half*>(Yv)[(size_t)j * ldy + n] = __float2half_rn(v);
        }
    }
}

int launch_gemm_wx_simt(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                        int ldy, int act, int y_is_f32, cudaStream_t st) {
    dim3 grid(ceil_div(N, 64), ceil_div(J, 64));
    if (y_is_f32)
        gemm_wx_simt_kernel<true><<<grid, 256, 0, st>>>(W, X, bias, Y, N, K, J, ldx, ldy, act);
    else
        gemm_wx_simt_kernel<false><<<grid, 256, 0, st>>>(W, X, bias, Y, N, K, J, ldx, ldy, act);
    return launch_status();
}

}  // namespace pimb200

// =============================================================================================
// C ABI
// =============================================================================================
using namespace pimb200;

extern "C" int pimb200_gemv_mv(const void* W, const void* x, const void* bias, void* y, int N, int K, int act,
                               void* stream) {
    if (!W || !x || !y || N <= 0 || K <= 0) return PIMB200_ERR_BAD_ARG;
    if (act != PIMB200_ACT_NONE && act != PIMB200_ACT_RELU) return PIMB200_ERR_BAD_ARG;
    return launch_gemv_mv(static_cast<const __half*>(W), static_cast<const __half*>(x),
                          static_cast<const __half*>(bias), static_cast<__half*>(y), N, K, act,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int pimb200_gemv_vm(const void* x, const void* A, const void* bias, void* y, int K, int N, int act,
                               void* stream) {
    if (!A || !x || !y || N <= 0 || K <= 0) return PIMB200_ERR_BAD_ARG;
    if (act != PIMB200_ACT_NONE && act != PIMB200_ACT_RELU) return PIMB200_ERR_BAD_ARG;
    return launch_gemv_vm(static_cast<const __half*>(x), static_cast<const __half*>(A),
                          static_cast<const __half*>(bias), static_cast<__half*>(y), K, N, act, true,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int pimb200_bmm_row(const void* x, const void* A, void* y, int k, int n, void* stream) {
    if (!A || !x || !y || n <= 0 || k <= 0) return PIMB200_ERR_BAD_ARG;
    // same kernel as VM without bias; k is a source-sentence length (tens of rows), so no K split
    return launch_gemv_vm(static_cast<const __half*>(x), static_cast<const __half*>(A), nullptr,
                          static_cast<__half*>(y), k, n, PIMB200_ACT_NONE, false, static_cast<cudaStream_t>(stream));
}

extern "C" int pimb200_dot_vv(const void* a, const void* b, void* y, int K, void* stream) {
    if (!a || !b || !y || K <= 0) return PIMB200_ERR_BAD_ARG;
    dot_vv_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __half*>(a),
                                                                   static_cast<const __half*>(b),
                                                                   static_cast<__half*>(y), K);
    return launch_status();
}

extern "C" int pimb200_add_f16(const void* A, const void* B, void* C, int m, int n, int broadcast_b, void* stream) {
    if (!A || !B || !C || m <= 0 || n <= 0) return PIMB200_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t total = (size_t)m * n;
    if (n % 8 == 0 && aligned16(A) && aligned16(B) && aligned16(C)) {
        size_t total8 = total / 8;
        size_t g = (total8 + 255) / 256;
        unsigned grid = (unsigned)(g > 148 * 8 ? 148 * 8 : g);
        add_f16_vec_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(A), static_cast<const uint4*>(B),
                                                 static_cast<uint4*>(C), total8, n / 8, broadcast_b ? 1 : 0);
    } else {
        size_t g = (total + 255) / 256;
        unsigned grid = (unsigned)(g > 148 * 8 ? 148 * 8 : g);
        add_f16_scalar_kernel<<<grid, 256, 0, st>>>(static_cast<const __half*>(A), static_cast<const __half*>(B),
                                                    static_cast<__half*>(C), total, n, broadcast_b ? 1 : 0);
    }
    return launch_status();
}

extern "C" int pimb200_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                               size_t rows, void* stream) {
    if (!dst || !src) return (row_bytes == 0 || rows == 0) ? PIMB200_OK : PIMB200_ERR_BAD_ARG;
    if (dst_pitch < row_bytes || src_pitch < row_bytes) return PIMB200_ERR_BAD_ARG;
    return launch_copy_2d(dst, dst_pitch, src, src_pitch, row_bytes, rows, static_cast<cudaStream_t>(stream));
}

extern "C" int pimb200_cat(void* dst, const void* const* src, const size_t* inner_bytes, int n_src, size_t outer,
                           void* stream) {
    if (!dst || !src || !inner_bytes || n_src <= 0) return PIMB200_ERR_BAD_ARG;
    size_t pitch = 0;
    for (int i = 0; i < n_src; ++i) pitch += inner_bytes[i];
    size_t off = 0;
    for (int i = 0; i < n_src; ++i) {
        if (inner_bytes[i] == 0) continue;  // empty operands are legal in aten::cat
        if (!src[i]) return PIMB200_ERR_BAD_ARG;
        int rc = launch_copy_2d(static_cast<unsigned char*>(dst) + off, pitch, src[i], inner_bytes[i], inner_bytes[i],
                                outer, static_cast<cudaStream_t>(stream));
        if (rc != PIMB200_OK) return rc;
        off += inner_bytes[i];
    }
    return PIMB200_OK;
}
