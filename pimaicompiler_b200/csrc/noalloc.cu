// pimb200_gemv_vm_static — the split-K vector-matrix product for callers that must not allocate.
//
// Some hosts cannot let a plug-in call cudaMalloc: an inference server that has given the whole device to its own
// arena (a cudaMalloc from inside the plug-in then fails, or is forbidden by the server's policy), or a latency
// critical loop that cannot afford the device-wide synchronisation an allocation implies.  pimb200_gemv_vm needs
// pimb200_init, which allocates a 16 MiB scratch with cudaMalloc.  This variant runs the same kernel with its
// scratch (fp32 partial sums of the K split and the per-tile ticket counters) in a file-scope device array that is
// part of the library image: every GPU that loads libpimb200.so holds it (about 1 MiB) until the process exits, and
// no call ever allocates or frees anything.
//
// The array's name is only a host-side stand-in in host code; the device address is looked up once per device
// with cudaGetSymbolAddress (with that device current) and passed to the kernel.
#include <mutex>

#include "common.cuh"

namespace pimb200 {
struct VmPlan {
    int lpr, tiles, splits, rows_per_split;
};
VmPlan plan_gemv_vm(int K, int N, size_t max_partial_floats, int max_tiles);
int launch_gemv_vm_with_scratch(const __half* x, const __half* A, const __half* bias, __half* y, int K, int N, int act,
                                const VmPlan& p, float* partials, unsigned int* tickets, cudaStream_t st);
}  // namespace pimb200

using namespace pimb200;

namespace {
constexpr int kStaticMaxN = PIMB200_VM_STATIC_MAX_N;
constexpr int kStaticMaxK = PIMB200_VM_STATIC_MAX_K;
constexpr size_t kStaticPartialFloats = (size_t)8 * kStaticMaxN;   // room for an 8-way K split at the widest N
constexpr int kStaticTiles = kStaticMaxN / 64;                     // narrowest column tile is 64 wide
constexpr size_t kStaticTicketBytes = (size_t)kStaticTiles * sizeof(unsigned int);
constexpr size_t kStaticBytes = kStaticPartialFloats * sizeof(float) + kStaticTicketBytes;

// [partials: kStaticPartialFloats floats][tickets: kStaticTiles counters]
static __device__ __align__(256) unsigned char g_vm_static_scratch[kStaticBytes];

std::mutex g_static_mu;
void* g_static_ptr[64];   // device address of the array, per device; filled on the first call on that device
}  // namespace

extern "C" int pimb200_gemv_vm_static(const void* x, const void* A, const void* bias, void* y, int K, int N, int act,
                                      void* stream) {
    if (!A || !x || !y || N <= 0 || K <= 0) return PIMB200_ERR_BAD_ARG;
    if (act != PIMB200_ACT_NONE && act != PIMB200_ACT_RELU) return PIMB200_ERR_BAD_ARG;
    // sizes beyond the fixed scratch, and layouts only the scratch-free generic kernel takes, are refused up front
    if (N > kStaticMaxN || K > kStaticMaxK) return PIMB200_ERR_UNSUPPORTED;
    if (N % 8 != 0 || !aligned16(A)) return PIMB200_ERR_UNSUPPORTED;
    int dev = 0;
    PIMB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return PIMB200_ERR_BAD_ARG;
    void* base = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static_ptr[dev]) {
            // first call on this device (it is the current one): resolve the array's device address
            void* p = nullptr;
            PIMB200_CUDA_TRY(cudaGetSymbolAddress(&p, g_vm_static_scratch));
            if (!p) return PIMB200_ERR_LAUNCH;
            g_static_ptr[dev] = p;
        }
        base = g_static_ptr[dev];
    }
    float* partials = static_cast<float*>(base);
    unsigned int* tickets = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(base) +
                                                            kStaticPartialFloats * sizeof(float));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const VmPlan p = plan_gemv_vm(K, N, kStaticPartialFloats, kStaticTiles);
    if (p.splits > 1) {
        // the array keeps whatever the previous call left: the ticket counters must start at zero
        PIMB200_CUDA_TRY(cudaMemsetAsync(tickets, 0, kStaticTicketBytes, st));
    }
    return launch_gemv_vm_with_scratch(static_cast<const __half*>(x), static_cast<const __half*>(A),
                                       static_cast<const __half*>(bias), static_cast<__half*>(y), K, N, act, p,
                                       partials, tickets, st);
}
