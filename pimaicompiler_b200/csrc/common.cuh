// Shared device/host helpers for the sm_100a kernels behind the pimb200 C ABI.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pimb200.h"

namespace pimb200 {

constexpr int kWarp = 32;
constexpr int kNumSmB200 = 148;

// ---- host side -------------------------------------------------------------
inline int cuda_status(cudaError_t e) {
    if (e == cudaSuccess) return PIMB200_OK;
    if (e == cudaErrorMemoryAllocation) return PIMB200_ERR_NO_MEMORY;
    return PIMB200_ERR_LAUNCH;
}
#define PIMB200_CUDA_TRY(expr)                                  \
    do {                                                        \
        cudaError_t _e = (expr);                                \
        if (_e != cudaSuccess) return ::pimb200::cuda_status(_e); \
    } while (0)

inline int launch_status() { return cuda_status(cudaGetLastError()); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// One product of a grouped launch: Y[J, N] = act(X[J, K] . W[N, K]^T + bias)
struct GemmProblem {
    const __half* W;
    const __half* X;
    const __half* bias;
    void* Y;
    int N, K, J, ldx, ldy, act, y_is_f32;
};

// Per-device scratch used by kernels that split one reduction across CTAs.
struct DeviceCtx {
    bool ready = false;
    float* splitk_partials = nullptr;   // [kSplitKMaxFloats]
    unsigned int* splitk_tickets = nullptr;  // [kSplitKMaxTiles], zero between calls
    int sm_count = kNumSmB200;
};
constexpr size_t kSplitKMaxFloats = size_t(1) << 22;  // 16 MiB of fp32 partial sums
constexpr int kSplitKMaxTiles = 4096;
DeviceCtx* current_ctx();  // nullptr when pimb200_init was not called for the current device

// ---- device side -----------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    // weights are read once per launch: keep them out of L1
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// Device status block of the kernels with bounded waits: word 0 is the sticky error code that *_last_status reads and
// clears; word 1 is the generation of the launch that gave up.  A launch aborts its waits only when word 1 carries its
// own generation (never 0), so one timed-out launch does not make later launches skip their work.
__device__ __forceinline__ bool status_aborted(const int* status, int gen) {
    return reinterpret_cast<const volatile int*>(status)[1] == gen;
}
__device__ __forceinline__ void status_raise(int* status, int gen, int code) {
    atomicExch(status, code);
    atomicExch(status + 1, gen);
}

__device__ __forceinline__ float2 h2f2(uint32_t v) {
    __half2 h = *reinterpret_cast<__half2*>(&v);
    return __half22float2(h);
}

// acc += dot(w[0..8), x[0..8)) with both operands packed as 8 halves
__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
    float2 a, b;
    a = h2f2(w.x); b = h2f2(x.x); acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
    a = h2f2(w.y); b = h2f2(x.y); acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
    a = h2f2(w.z); b = h2f2(x.z); acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
    a = h2f2(w.w); b = h2f2(x.w); acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
    return acc;
}

// acc += dot(w[0..8), xf[0..8)) with x already widened to fp32
__device__ __forceinline__ float dot8f(const uint4& w, const float* xf, float acc) {
    float2 a;
    a = h2f2(w.x); acc = fmaf(a.x, xf[0], acc); acc = fmaf(a.y, xf[1], acc);
    a = h2f2(w.y); acc = fmaf(a.x, xf[2], acc); acc = fmaf(a.y, xf[3], acc);
    a = h2f2(w.z); acc = fmaf(a.x, xf[4], acc); acc = fmaf(a.y, xf[5], acc);
    a = h2f2(w.w); acc = fmaf(a.x, xf[6], acc); acc = fmaf(a.y, xf[7], acc);
    return acc;
}

__device__ __forceinline__ void widen8(const uint4& x, float* xf) {
    float2 a;
    a = h2f2(x.x); xf[0] = a.x; xf[1] = a.y;
    a = h2f2(x.y); xf[2] = a.x; xf[3] = a.y;
    a = h2f2(x.z); xf[4] = a.x; xf[5] = a.y;
    a = h2f2(x.w); xf[6] = a.x; xf[7] = a.y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// exp and reciprocal both through the special-function unit (ex2.approx, rcp.approx: 1 ulp each, abs error of the
// result ~2e-7, far below the fp16 rounding of h).  The IEEE-rounded reciprocal (rcp.rn) expands to a Newton sequence
// with a guarded slow path; ten of those per LSTM cell ran back to back and made up most of the gate phase of the
// recurrence kernels.
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float sigmoidf_(float x) { return rcp_approx(1.0f + __expf(-x)); }
__device__ __forceinline__ float tanhf_(float x) {
    // tanh(x) = 2*sigmoid(2x) - 1
    return fmaf(2.0f, rcp_approx(1.0f + __expf(-2.0f * x)), -1.0f);
}

}  // namespace pimb200
