// Dense contraction  Y[j,n] = act(sum_k X[j,k] W[n,k] + b[n])  on the 5th-generation tensor cores.
//
// Used for the whole-sequence LSTM input projection (J = T*B rows), the encoder half of the RNN-T joint
// and the batched-stream linear layers (J = 8..128).  Both operands are K-major, so the weight matrix is
// the A operand (M = 128 weight rows per CTA) and the activations are the B operand (N = up to 128 rows
// of X per CTA, any multiple of 16):  D[m, j] = sum_k W[m0+m, k] X[j0+j, k], accumulated in fp32 in
// tensor memory.  TMEM lane = weight row, TMEM column = activation row, so the epilogue thread that owns
// weight row m adds bias[m] once and, for a fixed j, the 32 lanes of a warp store 32 consecutive
// elements of Y's row j.
//
// Persistent CTAs (one per SM) loop over output tiles, warp-specialised, two accumulator stages in tensor memory:
//   warp 0    TMA producer: cp.async.bulk.tensor (no multicast) of a [128 x 64] W tile and a [BN x 64] X tile
//             per stage, 128-byte swizzle, completion on the stage's "full" mbarrier
//   warp 1    allocates TMEM; one lane issues tcgen05.mma (kind::f16, M=128, N=BN, K=16) four times per
//             stage and commits the stage's "empty" mbarrier
//   warps 2-5 epilogue: tcgen05.ld 32 columns at a time, bias / ReLU / convert, coalesced stores
// Every mbarrier wait is bounded; when one runs out the kernel records an error in the status word,
// lets outstanding bulk copies land (bounded), frees its TMEM and returns.
// Shapes the TMA path cannot take (K or ldx not a multiple of 8, unaligned base) use the SIMT kernel.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc_common.cuh"

namespace pimb200 {

int launch_gemm_wx_simt(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                        int ldy, int act, int y_is_f32, cudaStream_t st);

namespace tc {

constexpr int BM = 128;            // weight rows per CTA (UMMA M)
constexpr int BN_MAX = 128;        // activation rows per CTA (UMMA N), runtime value in [16, 128]
constexpr int BK = 64;             // halves per stage along K = one 128-byte swizzle row
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_STAGE_BYTES = BN_MAX * BK * 2;    // 16 KiB
constexpr int THREADS = 192;                      // 6 warps
constexpr size_t SMEM_BYTES = (size_t)STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 1024 /*align*/ + 256 /*barriers*/;
// warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 = epilogue

struct GemmArgs {
    const __half* bias;   // [N] or NULL
    void* Y;
    int N, K, J, ldy, act, y_is_f32;
    int bn;               // activation rows per tile: multiple of 16 in [16, 128]
    int tmem_cols;        // power of two >= max(32, 2 * bn): two accumulator stages
    int m_tiles, j_tiles; // tiles along the weight rows and along the activation rows
    int* status;          // device status block: [0] sticky error code, [1] generation of the launch that gave up
    int gen;              // this launch's generation (never 0)
    int x_batch;          // > 0: X is [x_batch sequences][T steps][K] (batch-first) but the activation rows are numbered
                          //      time-major, row = t * x_batch + b; map_x is then a 3-D map (K, b, t) and bn % x_batch == 0
};

// Persistent: CTA b works on tiles b, b + gridDim.x, ...; consecutive tile numbers share the activation (j) block, so the
// X tile stays hot in L2 while the CTAs of a wave walk down the weight rows.  Two accumulator stages in tensor memory
// let the epilogue of one tile run under the MMAs of the next.
__global__ void __launch_bounds__(THREADS, 1)
gemm_wx_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmArgs a) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = smem;
    unsigned char* sB = smem + (size_t)STAGES * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + (size_t)STAGES * B_STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) accumulator full, [2S+2..2S+4) accumulator empty; then the TMEM base
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (a.K + BK - 1) / BK;
    const int n_tiles = a.m_tiles * a.j_tiles;
    const volatile int* abort_flag = a.status + 1;   // generation of the launch that gave up

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(accf0 + 8 * s, 1);
            mbar_init(acce0 + 8 * s, 4);   // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)a.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    bool failed = false;

    if (warp == 0) {
        // ---------------- TMA producer: one continuous stream of k-blocks over all tiles of this CTA ----------------
        if (lane == 0) {
            const uint32_t stage_bytes = (uint32_t)A_STAGE_BYTES + (uint32_t)a.bn * BK * 2;
            int issued = 0;  // k-blocks issued so far = position in the shared-memory ring
            for (int tile = blockIdx.x; tile < n_tiles && !failed; tile += gridDim.x) {
                const int m0 = (tile % a.m_tiles) * BM, j0 = (tile / a.m_tiles) * a.bn;
                const int t0 = a.x_batch > 0 ? j0 / a.x_batch : 0;   // first timestep of the tile (once per tile)
                for (int kb = 0; kb < kblocks; ++kb, ++issued) {
                    const int s = issued % STAGES;
                    const uint32_t it = (uint32_t)(issued / STAGES);
                    if (!mbar_wait(empty0 + 8 * s, (it & 1) ^ 1, abort_flag, a.gen)) { failed = true; break; }
                    mbar_expect_tx(full0 + 8 * s, stage_bytes);
                    tma_load_2d(smem_u32(sA + (size_t)s * A_STAGE_BYTES), &map_w, full0 + 8 * s, kb * BK, m0);
                    if (a.x_batch > 0)   // bn / x_batch whole timesteps of all sequences, sequence index fastest
                        tma_load_3d(smem_u32(sB + (size_t)s * B_STAGE_BYTES), &map_x, full0 + 8 * s, kb * BK, 0, t0);
                    else
                        tma_load_2d(smem_u32(sB + (size_t)s * B_STAGE_BYTES), &map_x, full0 + 8 * s, kb * BK, j0);
                }
            }
            if (failed) {
                status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
                // let the copies already issued land before the CTA gives its shared memory back
                const int first = issued > STAGES ? issued - STAGES : 0;
                for (int q = first; q < issued; ++q) {
                    const int s = q % STAGES;
                    for (uint32_t i = 0; i < (1u << 20); ++i)
                        if (mbar_try_wait(full0 + 8 * s, (uint32_t)(q / STAGES) & 1)) break;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: D = f32, A = B = f16, both K-major, N = bn, M = 128
            const uint32_t idesc = (1u << 4) | ((uint32_t)(a.bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int consumed = 0, local = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !failed; tile += gridDim.x, ++local) {
                const int as = local & 1;                          // accumulator stage
                const uint32_t ait = (uint32_t)(local >> 1);        // how often this stage has been used before
                if (!mbar_wait(acce0 + 8 * as, (ait & 1) ^ 1, abort_flag, a.gen)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * a.bn);
                for (int kb = 0; kb < kblocks; ++kb, ++consumed) {
                    const int s = consumed % STAGES;
                    const uint32_t it = (uint32_t)(consumed / STAGES);
                    if (!mbar_wait(full0 + 8 * s, it & 1, abort_flag, a.gen)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t adesc = make_smem_desc(smem_u32(sA + (size_t)s * A_STAGE_BYTES));
                    const uint64_t bdesc = make_smem_desc(smem_u32(sB + (size_t)s * B_STAGE_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // advance 16 halves = 32 bytes inside the swizzle row: +2 in the descriptor's 16-byte units
                        umma_f16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                                 (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty0 + 8 * s);  // the stage is free once these MMAs have read it
                }
                umma_commit(accf0 + 8 * as);      // this tile's accumulator is complete once everything above retires
            }
            if (failed) {
                status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
                umma_commit(accf0);               // wake epilogue warps; they see the status word and leave
                umma_commit(accf0 + 8);
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----------------
        const int q = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int as = local & 1;
            const uint32_t ait = (uint32_t)(local >> 1);
            const int m0 = (tile % a.m_tiles) * BM, j0 = (tile / a.m_tiles) * a.bn;
            const int m = m0 + q * 32 + lane;
            bool ok = mbar_wait(accf0 + 8 * as, ait & 1, abort_flag, a.gen);
            if (!ok) status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!ok || *abort_flag == a.gen) break;
            const float bv = (a.bias && m < a.N) ? __half2float(a.bias[m]) : 0.f;
            const float lo = a.act == PIMB200_ACT_RELU ? 0.f : -INFINITY;   // v = max(v, lo): ReLU without a branch
            const int j_end = a.J < j0 + a.bn ? a.J : j0 + a.bn;            // first activation row past this tile
            // One warp per scheduler runs this loop with nothing to hide instruction latency behind, so the common case
            // (all 32 columns of a chunk inside the matrix) carries no per-element checks or index arithmetic: a
            // running pointer, one add, one max, one store.
            float* yf = static_cast<float*>(a.Y) + (size_t)j0 * a.ldy + m;
            __half* yh = static_cast<__half*>(a.Y) + (size_t)j0 * a.ldy + m;
            for (int c0 = 0; c0 < a.bn; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * a.bn + c0), r);
                if (m < a.N) {
                    if (j0 + c0 + 32 <= j_end) {
                        if (a.y_is_f32) {
#pragma unroll
                            for (int c = 0; c < 32; ++c) yf[(size_t)c * a.ldy] = fmaxf(__uint_as_float(r[c]) + bv, lo);
                        } else {
#pragma unroll
                            for (int c = 0; c < 32; ++c)
                                yh[(size_t)c * a.ldy] = __float2half_rn(fmaxf(__uint_as_float(r[c]) + bv, lo));
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            if (j0 + c0 + c < j_end) {
                                const float v = fmaxf(__uint_as_float(r[c]) + bv, lo);
                                if (a.y_is_f32) yf[(size_t)c * a.ldy] = v;
                                else yh[(size_t)c * a.ldy] = __float2half_rn(v);
                            }
                        }
                    }
                }
                yf += (size_t)32 * a.ldy;
                yh += (size_t)32 * a.ldy;
            }
            // this warp is done reading the stage: hand it back to the MMA issuer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acce0 + 8 * as) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)a.tmem_cols)
                     : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static std::mutex g_mu;
static EncodeTiledFn g_encode = nullptr;
static bool g_encode_tried = false;
constexpr int kMaxDevices = 64;
static int* g_status[kMaxDevices];       // per device: {sticky error code, generation of the launch that gave up}
static bool g_attr_set[kMaxDevices];     // cudaFuncSetAttribute is per device
static int g_gen = 0;                    // launch generation, never 0

static EncodeTiledFn get_encode() {
    if (g_encode_tried) return g_encode;
    g_encode_tried = true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    else
        cudaGetLastError();
    return g_encode;
}

static bool encode_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                      uint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// X as [batch][steps][K] (row (b, t) at (b*steps + t) * ldx), tiles of box_t timesteps x all `batch` sequences
static bool encode_x_time_major(CUtensorMap* map, const void* base, uint64_t batch, uint64_t steps, uint64_t cols,
                                uint64_t ldx_bytes, uint32_t box_t) {
    const cuuint64_t dims[3] = {cols, batch, steps};
    const cuuint64_t strides[2] = {steps * ldx_bytes, ldx_bytes};
    const cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)batch, box_t};
    const cuuint32_t estr[3] = {1, 1, 1};
    return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// returns PIMB200_ERR_UNSUPPORTED when the shape must take the SIMT kernel.  x_batch > 0: X is batch-first
// [x_batch][J / x_batch][K] and the output rows are numbered time-major (row = t * x_batch + b).
static int launch(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx, int ldy,
                  int act, int y_is_f32, cudaStream_t st, int x_batch) {
    if (K % 8 != 0 || ldx % 8 != 0 || !aligned16(W) || !aligned16(X)) return PIMB200_ERR_UNSUPPORTED;
    int dev = 0;
    PIMB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return PIMB200_ERR_UNSUPPORTED;
    int* status = nullptr;
    int gen = 0;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!get_encode()) return PIMB200_ERR_UNSUPPORTED;
        if (!g_status[dev]) {
            PIMB200_CUDA_TRY(cudaMalloc(&g_status[dev], 2 * sizeof(int)));
            PIMB200_CUDA_TRY(cudaMemset(g_status[dev], 0, 2 * sizeof(int)));
        }
        status = g_status[dev];
        if (!g_attr_set[dev]) {
            PIMB200_CUDA_TRY(cudaFuncSetAttribute(gemm_wx_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)SMEM_BYTES));
            g_attr_set[dev] = true;
        }
        if (++g_gen == 0) g_gen = 1;
        gen = g_gen;
    }
    GemmArgs a;
    a.gen = gen;
    a.bias = bias; a.Y = Y; a.N = N; a.K = K; a.J = J; a.ldy = ldy; a.act = act; a.y_is_f32 = y_is_f32;
    a.bn = J >= BN_MAX ? BN_MAX : ((J + 15) / 16) * 16;
    a.x_batch = 0;
    if (x_batch > 0) {
        if (J % x_batch != 0 || a.bn % x_batch != 0 || x_batch > 256) return PIMB200_ERR_UNSUPPORTED;
        a.x_batch = x_batch;
    }
    // two stages of bn columns; the epilogue reads 32 columns at a time, so the second stage needs its length rounded up
    const int need_cols = a.bn + ((a.bn + 31) / 32) * 32;
    a.tmem_cols = need_cols <= 32 ? 32 : (need_cols <= 64 ? 64 : (need_cols <= 128 ? 128 : 256));
    a.m_tiles = ceil_div(N, BM);
    a.j_tiles = ceil_div(J, a.bn);
    a.status = status;
    CUtensorMap map_w, map_x;
    if (!encode_2d(&map_w, W, (uint64_t)N, (uint64_t)K, (uint64_t)K * 2, BM)) return PIMB200_ERR_UNSUPPORTED;
    if (a.x_batch > 0) {
        if (!encode_x_time_major(&map_x, X, (uint64_t)x_batch, (uint64_t)(J / x_batch), (uint64_t)K, (uint64_t)ldx * 2,
                                 (uint32_t)(a.bn / x_batch)))
            return PIMB200_ERR_UNSUPPORTED;
    } else if (!encode_2d(&map_x, X, (uint64_t)J, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)a.bn)) {
        return PIMB200_ERR_UNSUPPORTED;
    }
    const long tiles = (long)a.m_tiles * a.j_tiles;
    int sms = kNumSmB200;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int)(tiles < sms ? tiles : sms);
    gemm_wx_tc_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(map_w, map_x, a);
    return launch_status();
}

}  // namespace tc

static int g_force_simt = 0;

int launch_gemm_wx_skinny(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                          int ldy, int act, int y_is_f32, cudaStream_t st);

// Router of the dense contraction: up to 32 activation rows stream W on every SM (HBM-bound, like the GEMV); more rows
// go to the tcgen05 kernel; shapes neither takes (unaligned operands, K not a multiple of 8) to the SIMT kernel.
int launch_gemm_wx(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                   int ldy, int act, int y_is_f32, cudaStream_t st) {
    if (!g_force_simt) {
        const int rs = launch_gemm_wx_skinny(W, X, bias, Y, N, K, J, ldx, ldy, act, y_is_f32, st);
        if (rs != PIMB200_ERR_UNSUPPORTED) return rs;
        const int rc = tc::launch(W, X, bias, Y, N, K, J, ldx, ldy, act, y_is_f32, st, 0);
        if (rc != PIMB200_ERR_UNSUPPORTED) return rc;
    }
    return launch_gemm_wx_simt(W, X, bias, Y, N, K, J, ldx, ldy, act, y_is_f32, st);
}

// Y[t * batch + b, :] = X[b, t, :] . W^T for a batch-first X [batch][J / batch][K]: the projection of a batch-first
// sequence tensor written in time-major row order.  Tensor-core path only; PIMB200_ERR_UNSUPPORTED when the shape does
// not allow it (the caller then projects in the input's own row order).
int launch_gemm_wx_time_major(const __half* W, const __half* X, void* Y, int N, int K, int J, int ldx, int ldy, int batch,
                              cudaStream_t st) {
    if (g_force_simt || batch <= 0) return PIMB200_ERR_UNSUPPORTED;
    return tc::launch(W, X, nullptr, Y, N, K, J, ldx, ldy, PIMB200_ACT_NONE, 1, st, batch);
}

}  // namespace pimb200

// A/B switch for profiling: 1 = always the SIMT kernel.
extern "C" int pimb200_gemm_force_simt(int on) {
    pimb200::g_force_simt = on ? 1 : 0;
    return PIMB200_OK;
}

// Status word of the tensor-core GEMM on the current device: 0, or PIMB200_ERR_TIMEOUT when one of its bounded
// waits gave up since the last call.  Synchronises the device.
extern "C" int pimb200_gemm_last_status(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return PIMB200_ERR_LAUNCH;
    if (dev < 0 || dev >= pimb200::tc::kMaxDevices) return PIMB200_OK;
    int* p = nullptr;
    {
        std::lock_guard<std::mutex> lk(pimb200::tc::g_mu);
        p = pimb200::tc::g_status[dev];
    }
    if (!p) return PIMB200_OK;
    int v = 0;
    if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return PIMB200_ERR_LAUNCH;
    if (v != 0) cudaMemset(p, 0, sizeof(int));
    return v;
}
