// Library lifetime, per-device scratch and the remaining C-ABI entry points.
#include <mutex>

#include "common.cuh"

namespace pimb200 {

int launch_gemm_wx(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                   int ldy, int act, int y_is_f32, cudaStream_t st);

static std::mutex g_ctx_mutex;
static DeviceCtx g_ctx[64];

DeviceCtx* current_ctx() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_ctx_mutex);
    return g_ctx[dev].ready ? &g_ctx[dev] : nullptr;
}

}  // namespace pimb200

using namespace pimb200;

extern "C" const char* pimb200_status_string(int status) {
    switch (status) {
        case PIMB200_OK: return "ok";
        case PIMB200_ERR_BAD_ARG: return "bad argument";
        case PIMB200_ERR_UNSUPPORTED: return "unsupported shape";
        case PIMB200_ERR_LAUNCH: return "CUDA launch/runtime failure";
        case PIMB200_ERR_TIMEOUT: return "bounded device-side wait ran out";
        case PIMB200_ERR_NOT_INIT: return "pimb200_init not called for this device";
        case PIMB200_ERR_NO_MEMORY: return "device allocation failed";
        default: return "unknown status";
    }
}

extern "C" int pimb200_init(int device) {
    if (device < 0 || device >= 64) return PIMB200_ERR_BAD_ARG;
    int count = 0;
    PIMB200_CUDA_TRY(cudaGetDeviceCount(&count));
    if (device >= count) return PIMB200_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lk(g_ctx_mutex);
    DeviceCtx& c = g_ctx[device];
    if (c.ready) return PIMB200_OK;
    int prev = 0;
    PIMB200_CUDA_TRY(cudaGetDevice(&prev));
    PIMB200_CUDA_TRY(cudaSetDevice(device));
    int rc = PIMB200_OK;
    do {
        if ((rc = cuda_status(cudaMalloc(&c.splitk_partials, kSplitKMaxFloats * sizeof(float)))) != PIMB200_OK) break;
        if ((rc = cuda_status(cudaMalloc(&c.splitk_tickets, kSplitKMaxTiles * sizeof(unsigned int)))) != PIMB200_OK) break;
        if ((rc = cuda_status(cudaMemset(c.splitk_tickets, 0, kSplitKMaxTiles * sizeof(unsigned int)))) != PIMB200_OK) break;
        cudaDeviceGetAttribute(&c.sm_count, cudaDevAttrMultiProcessorCount, device);
        if ((rc = cuda_status(cudaDeviceSynchronize())) != PIMB200_OK) break;
        c.ready = true;
    } while (0);
    if (rc != PIMB200_OK) {
        cudaFree(c.splitk_partials);
        cudaFree(c.splitk_tickets);
        c = DeviceCtx();
    }
    cudaSetDevice(prev);
    return rc;
}

extern "C" int pimb200_shutdown(int device) {
    if (device < 0 || device >= 64) return PIMB200_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lk(g_ctx_mutex);
    DeviceCtx& c = g_ctx[device];
    if (!c.ready) return PIMB200_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(device);
    cudaDeviceSynchronize();
    cudaFree(c.splitk_partials);
    cudaFree(c.splitk_tickets);
    c = DeviceCtx();
    cudaSetDevice(prev);
    return PIMB200_OK;
}

extern "C" int pimb200_gemm_wx(const void* W, const void* X, const void* bias, void* Y, int N, int K, int J, int ldx,
                               int ldy, int act, int y_is_f32, void* stream) {
    if (!W || !X || !Y || N <= 0 || K <= 0 || J <= 0 || ldx < K || ldy < N) return PIMB200_ERR_BAD_ARG;
    if (act != PIMB200_ACT_NONE && act != PIMB200_ACT_RELU) return PIMB200_ERR_BAD_ARG;
    return launch_gemm_wx(static_cast<const __half*>(W), static_cast<const __half*>(X),
                          static_cast<const __half*>(bias), Y, N, K, J, ldx, ldy, act, y_is_f32,
                          static_cast<cudaStream_t>(stream));
}

namespace pimb200 {
int launch_gemm_wx_grouped(const GemmProblem* pr, int n, cudaStream_t st);
}

extern "C" int pimb200_gemm_wx_grouped(const pimb200_gemm_problem* problems, int n, void* stream) {
    if (n == 0) return PIMB200_OK;
    if (!problems || n < 0) return PIMB200_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < n; ++i) {
        const pimb200_gemm_problem& q = problems[i];
        if (!q.W || !q.X || !q.Y || q.N <= 0 || q.K <= 0 || q.J <= 0 || q.ldx < q.K || q.ldy < q.N) return PIMB200_ERR_BAD_ARG;
        if (q.act != PIMB200_ACT_NONE && q.act != PIMB200_ACT_RELU) return PIMB200_ERR_BAD_ARG;
    }
    // groups of up to 8 problems per launch; a group with a shape the few-row kernel does not take runs one by one
    for (int i0 = 0; i0 < n; i0 += 8) {
        const int m = n - i0 < 8 ? n - i0 : 8;
        GemmProblem g[8];
        for (int i = 0; i < m; ++i) {
            const pimb200_gemm_problem& q = problems[i0 + i];
            g[i] = GemmProblem{static_cast<const __half*>(q.W), static_cast<const __half*>(q.X), static_cast<const __half*>(q.bias),
                               q.Y, q.N, q.K, q.J, q.ldx, q.ldy, q.act, q.y_is_f32};
        }
        int rc = launch_gemm_wx_grouped(g, m, st);
        if (rc == PIMB200_ERR_UNSUPPORTED) {
            for (int i = 0; i < m; ++i) {
                rc = launch_gemm_wx(g[i].W, g[i].X, g[i].bias, g[i].Y, g[i].N, g[i].K, g[i].J, g[i].ldx, g[i].ldy, g[i].act,
                                    g[i].y_is_f32, st);
                if (rc != PIMB200_OK) return rc;
            }
        } else if (rc != PIMB200_OK) {
            return rc;
        }
    }
    return PIMB200_OK;
}
