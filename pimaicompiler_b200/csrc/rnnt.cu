// Device-resident RNN-T greedy decode.
//
// The reference runs the whole RNN-T model as one interpreted TorchScript graph: the encoder LSTMs are
// aten::lstm nodes, and the greedy loop is a prim::Loop walked by the host
// (runtime/source/executor/stream_executor.cpp:153-186, prim_ops_executor.cpp:744-922) that costs, per
// decoded frame, an embedding lookup with a device->host sync (aten_ops_executor.cpp:1276-1287), two
// seq_len==1 aten::lstm calls, the split joint addmm pair + ReLU + addmm (remove_cat_for_addmm.h:77-79,
// fuse_activation.cpp:88-93) and an argmax read back by the host.  Here the encoder is the fused LSTM of
// lstm.cu plus one dense GEMM for the encoder half of the joint, and the whole greedy loop is ONE kernel:
// a thread-block cluster keeps the prediction network and the joint in shared memory, exchanges hidden
// states through distributed shared memory, and every CTA takes the blank/emit decision redundantly from
// identical inputs, so no host round trip and no decision broadcast is needed.
//
// Model (sizes are run-time arguments; the defaults are the benchmark's):
//   enc  : LSTM(F -> EH, pre_layers) -> stack `stack` frames -> LSTM(stack*EH -> EH, post_layers)
//   pred : Embedding(V, PH) -> LSTM(PH -> PH, 2 layers); start-of-sequence input is the blank row
//   joint: Linear(EH+PH -> JH) -> ReLU -> Linear(JH -> V); greedy, at most one symbol per frame
#include <cooperative_groups.h>

#include <mutex>
#include <vector>

#include "common.cuh"
#include "pimb200_rnnt.h"

namespace cg = cooperative_groups;
using namespace pimb200;

namespace pimb200 {
int launch_gemm_wx(const __half* W, const __half* X, const __half* bias, void* Y, int N, int K, int J, int ldx,
                   int ldy, int act, int y_is_f32, cudaStream_t st);
}
namespace pimb200 {
void lstm_pack_matrix(const __half* src, __half* dst, int H, int cols, cudaStream_t st);
void lstm_pack_bias(const __half* b_ih, const __half* b_hh, float* dst, int H, cudaStream_t st);
}

__global__ void rnnt_add_bias_rows_kernel(float* __restrict__ P0, const float* __restrict__ bias, int n, int rows) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n * rows) P0[i] += bias[i % n];
}
// W1p[JH][PH] -> fragment order for clusters of C CTAs (JP = JH / C rows per CTA, PH / 64 k-tiles per K quarter): word
// ((((cta * MTJ + mt) * 4 + kq) * NK + i) * 32 + lane) * 4 + r holds the two halves at row cta*JP + mt*16 + lane/4 +
// (r & 1) * 8, columns (kq*NK + i)*16 + 2*(lane % 4) + (r >> 1) * 8 ...+1: register r of that lane's A operand.  A warp
// then reads one k-tile of its operand as 512 contiguous bytes instead of 128 scattered words.
__global__ void rnnt_pack_w1p_frags_kernel(const __half* __restrict__ W1p, uint32_t* __restrict__ out, int JH, int PH, int C) {
    const int NK = PH / 64, JP = JH / C, MTJ = JP / 16;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)JH * PH / 2) return;
    size_t w = idx;
    const int r = (int)(w & 3); w >>= 2;
    const int lane = (int)(w & 31); w >>= 5;
    const int i = (int)(w % NK); w /= NK;
    const int kq = (int)(w & 3); w >>= 2;
    const int mt = (int)(w % MTJ); w /= MTJ;
    const int cta = (int)w;
    const int row = cta * JP + mt * 16 + (lane >> 2) + (r & 1) * 8;
    const int col = (kq * NK + i) * 16 + 2 * (lane & 3) + (r >> 1) * 8;
    out[idx] = *reinterpret_cast<const uint32_t*>(W1p + (size_t)row * PH + col);
}
__global__ void rnnt_widen_kernel(const __half* __restrict__ src, float* __restrict__ dst, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __half2float(src[i]);
}

struct GreedyArgs {
    // per-utterance inputs/outputs
    const float* E;        // [n_utts][Tp][JH]  encoder half of the joint, bias b1 included
    int* tokens;           // [n_utts][Tp]
    int* n_tokens;         // [n_utts]
    float* logits;         // optional [n_utts][Tp][V]
    int n_utts, Tp;
    // prediction network (gate-interleaved packed rows u*4+g)
    const float* P0;       // [V][4PH]  W_ih0 . emb[k] + b_ih0 + b_hh0
    const __half* Whh0;    // [4PH][PH]
    const __half* Wih1;    // [4PH][PH]
    const __half* Whh1;    // [4PH][PH]
    const float* bias1;    // [4PH]
    // joint
    const __half* W1p;     // [JH][PH]   prediction half of the first joint matrix
    const uint4* W1pf;     // the same matrix in the order the tensor-core kernel's threads consume it (or NULL):
                           // [CTA][m-tile][K quarter][k-tile][lane] x the four A registers of an m16n8k16 product
    const __half* W2;      // [V][JH]
    const float* b2;       // [V]
    int PH, JH, V, blank;
    int smem_mask;         // bit i set = matrix i (Whh0, Wih1, Whh1, W1p, W2) is staged in shared memory
    long long* trace;      // optional diagnostics: 8 clocks per frame of utterance 0 (cluster 0, CTA 0)
    int* status;           // device status block: [0] sticky error code, [1] generation of the launch that gave up
    int gen;               // generation of this launch (never 0)
    int poll_limit;        // bound of every wait on an exchange barrier, in polls
};

// ---- all-to-all exchange inside a cluster without cluster-wide barriers ------------------------------------
// A cluster barrier after remote stores costs the sender a release of those stores (a round trip to every peer)
// before it may even arrive.  Here every value travels as st.async: the store itself reports its bytes to an mbarrier
// in the RECEIVING CTA, which therefore learns of the arrival one way, and the sender never waits.  Each exchange
// has two mbarriers used alternately: a peer can be at most one exchange ahead (it needs this CTA's contribution to
// pass its own wait), so bytes of use k+1 never meet a barrier still counting use k.
constexpr long long kGreedyWaitCycles = 4000000000ll;   // about two seconds
constexpr int kGreedyPollLimit = 1 << 26;
__device__ __forceinline__ uint32_t g_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t g_mapa(uint32_t addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void g_st_async_b32(uint32_t dst, uint32_t v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(dst), "r"(v),
                 "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void g_st_async_v2(uint32_t dst, const uint2& v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(dst),
                 "r"(v.x), "r"(v.y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void g_st_async_v4(uint32_t dst, const uint4& v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(dst),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void g_xbar_init(uint32_t bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void g_xbar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool g_xbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded: false = gave up (poll or time limit), or another CTA of this launch already did
__device__ __forceinline__ bool g_xbar_wait(uint32_t bar, uint32_t parity, const int* status, int gen, int limit) {
    if (g_xbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (int i = 1; i < limit; ++i) {
        if (g_xbar_try(bar, parity)) return true;
        if ((i & 255) == 0 && (status_aborted(status, gen) || clock64() - t0 > kGreedyWaitCycles)) return false;
    }
    return false;
}

constexpr int kGreedyThreads = 512;
constexpr int kGreedyWarps = kGreedyThreads / 32;
constexpr int kMaxRowsPerWarp = 8;   // rows of one phase a warp may own (rows / 16 warps, rounded up)

// z[i] += W[row_i, :] . h for the rows row_i = warp + 16*i of a [rows x K] matrix: all rows of a warp
// advance together, so their loads and FMA chains are independent and overlap
template <int NR>
__device__ __forceinline__ void rows_dot(const __half* __restrict__ W, int rows, int K, const __half* __restrict__ h,
                                         int warp, int lane, float* z) {
    const int K8 = K >> 3;
    const uint4* h4 = reinterpret_cast<const uint4*>(h);
    for (int c = lane; c < K8; c += 32) {
        float xf[8];
        widen8(h4[c], xf);
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int r = warp + kGreedyWarps * i;
            if (r < rows) z[i] = dot8f(reinterpret_cast<const uint4*>(W + (size_t)r * K)[c], xf, z[i]);
        }
    }
}
template <int NR>
__device__ __forceinline__ void rows_reduce(float* z) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < NR; ++i) z[i] += __shfl_xor_sync(0xffffffffu, z[i], o);
}

// NRG / NRJ / NRV = rows per warp of the gate phases, the joint slice and the vocabulary.  XB = the three exchanges of
// an evaluation travel as st.async with one mbarrier per receiver (needs PH % C == 0 and an even number of units per
// CTA: the state moves in 32-bit words); otherwise plain remote stores and cluster barriers.
template <int NRG, int NRJ, int NRV, bool XB>
__global__ void __launch_bounds__(kGreedyThreads, 1) rnnt_greedy_kernel(GreedyArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    const int C = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int cluster_id = blockIdx.x / C, n_clusters = gridDim.x / C;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int nthr = kGreedyThreads;
    const int PH = a.PH, JH = a.JH, V = a.V;
    const int UP = (PH + C - 1) / C, u0 = rank * UP, nu = max(0, min(UP, PH - u0));
    const int JP = (JH + C - 1) / C, j0 = rank * JP, nj = max(0, min(JP, JH - j0));

    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned char* sp = smem_raw;
    auto carve = [&](size_t bytes) {
        unsigned char* p = sp;
        sp += (bytes + 15) & ~size_t(15);
        return p;
    };
    __half* h0buf = reinterpret_cast<__half*>(carve((size_t)2 * PH * 2));   // [2][PH]
    __half* h1buf = reinterpret_cast<__half*>(carve((size_t)2 * PH * 2));   // [2][PH]
    float* Pj = reinterpret_cast<float*>(carve((size_t)JH * 4));            // pred half of the joint
    __half* zs = reinterpret_cast<__half*>(carve((size_t)JH * 2));          // relu(E + Pj), fp16 like the op's output
    float* zrow = reinterpret_cast<float*>(carve((size_t)4 * UP * 4));      // gate pre-activations of my units
    float* lg = reinterpret_cast<float*>(carve((size_t)(V + 1) * 4));       // logits
    float* b2s = reinterpret_cast<float*>(carve((size_t)V * 4));            // output bias
    float* bias1s = reinterpret_cast<float*>(carve((size_t)4 * UP * 4));    // layer-1 bias of my rows
    float* P0s = reinterpret_cast<float*>(carve((size_t)V * 4 * UP * 4));   // [V][4UP] layer-0 input term of my rows
    __half* hst = reinterpret_cast<__half*>(carve((size_t)UP * 2));         // new hidden values of my units, before they travel
    const uint32_t xbar0 = g_smem_u32(carve(6 * 8));                        // exchange barriers [exchange 0..2][use & 1]
    const size_t slice = (size_t)4 * UP * PH * 2;
    // weight slices: staged in shared memory when they fit, else read in place (L2)
    const __half* Whh0 = a.Whh0 + (size_t)u0 * 4 * PH;
    const __half* Wih1 = a.Wih1 + (size_t)u0 * 4 * PH;
    const __half* Whh1 = a.Whh1 + (size_t)u0 * 4 * PH;
    const __half* W1p = a.W1p + (size_t)j0 * PH;
    const __half* W2 = a.W2;
    auto stage = [&](const __half* g, size_t halves, size_t cap_bytes) {
        __half* s = reinterpret_cast<__half*>(carve(cap_bytes));
        const uint4* g4 = reinterpret_cast<const uint4*>(g);
        uint4* s4 = reinterpret_cast<uint4*>(s);
        for (size_t i = tid; i < halves / 8; i += nthr) s4[i] = __ldg(g4 + i);
        return (const __half*)s;
    };
    if (a.smem_mask & 1) Whh0 = stage(Whh0, (size_t)4 * nu * PH, slice);
    if (a.smem_mask & 2) Wih1 = stage(Wih1, (size_t)4 * nu * PH, slice);
    if (a.smem_mask & 4) Whh1 = stage(Whh1, (size_t)4 * nu * PH, slice);
    if (a.smem_mask & 8) W1p = stage(W1p, (size_t)nj * PH, (size_t)JP * PH * 2);
    if (a.smem_mask & 16) W2 = stage(W2, (size_t)V * JH, (size_t)V * JH * 2);
    for (int i = tid; i < V; i += nthr) b2s[i] = a.b2[i];
    for (int i = tid; i < 4 * nu; i += nthr) bias1s[i] = a.bias1[(size_t)u0 * 4 + i];
    for (int i = tid; i < V * 4 * nu; i += nthr) {
        const int k = i / (4 * nu), r = i - k * 4 * nu;
        P0s[k * 4 * UP + r] = a.P0[(size_t)k * 4 * PH + (size_t)u0 * 4 + r];
    }

    // Gate threads.  With cluster barriers: thread (j, d) = (tid / C, tid % C) keeps the cell state of unit u0+j and
    // writes the new hidden value into CTA d, so the C copies of a unit are produced by C threads in parallel (same
    // inputs, same result).  With st.async: thread j < nu owns unit u0+j; the values are staged and sent as words.
    const int gj = XB ? tid : tid / C, gd = XB ? 0 : tid - gj * C;
    const bool gate_thread = gj < nu;
    float c_l0 = 0.f, c_l1 = 0.f;  // fp32 cell states for the whole utterance
    long long* trp = nullptr;
    uint32_t n_eval = 0;    // evaluations of this launch: use n_eval of an exchange takes barrier n_eval & 1, phase n_eval >> 1
    bool dead = false;      // a wait of this thread ran out: no more waits, no more sends
    if (XB && tid == 0) {
        for (int i = 0; i < 6; ++i) g_xbar_init(xbar0 + 8u * i);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    auto xwait = [&](int x) {
        if (dead) return;
        if (!g_xbar_wait(xbar0 + 8u * (2 * x + (n_eval & 1u)), (n_eval >> 1) & 1u, a.status, a.gen, a.poll_limit)) {
            dead = true;
            status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
        }
    };
    // my units' staged values -> the same place of `dst_local` in every CTA, one 32-bit word a thread
    auto send_state = [&](__half* dst_local, int x) {
        const int W = nu >> 1;
        if (tid < C * W && !dead) {
            const int d = tid / W, w = tid - d * W;
            g_st_async_b32(g_mapa(g_smem_u32(dst_local + u0) + 4u * w, d), reinterpret_cast<const uint32_t*>(hst)[w],
                           g_mapa(xbar0 + 8u * (2 * x + (n_eval & 1u)), d));
        }
    };

    // One evaluation of the prediction network for input token `tok`, from the state left by the previous
    // evaluation (buffers of parity (e+1)&1), into buffers of parity e&1; then the pred half of the joint.
    float zp0[NRG], zp1[NRG];  // Whh0 . h0 and Whh1 . h1 of the coming evaluation, per-lane partial sums
    auto pred_eval = [&](int tok, int e) {
        __half* h0new_local = h0buf + (size_t)(e & 1) * PH;
        __half* h1new_local = h1buf + (size_t)(e & 1) * PH;
        if (XB && tid == 0) {   // what this CTA receives in the three exchanges of this evaluation
            const uint32_t b = n_eval & 1u;
            g_xbar_expect(xbar0 + 8u * b, PH * 2);
            g_xbar_expect(xbar0 + 8u * (2 + b), PH * 2);
            g_xbar_expect(xbar0 + 8u * (4 + b), JH * 4);
        }
        float z[NRG];
        // layer 0: the state product was made at the end of the previous evaluation
#pragma unroll
        for (int i = 0; i < NRG; ++i) z[i] = zp0[i];
        rows_reduce<NRG>(z);
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < NRG; ++i) {
                const int r = warp + kGreedyWarps * i;
                if (r < 4 * nu) zrow[r] = z[i] + P0s[tok * 4 * UP + r];
            }
        }
        __syncthreads();
        if (trp && tid == 0) trp[3] = clock64();
        if (gate_thread) {
            const float zi = zrow[gj * 4], zf = zrow[gj * 4 + 1], zg = zrow[gj * 4 + 2], zo = zrow[gj * 4 + 3];
            c_l0 = sigmoidf_(zf) * c_l0 + sigmoidf_(zi) * tanhf_(zg);
            const __half hv = __float2half_rn(sigmoidf_(zo) * tanhf_(c_l0));
            if (XB) hst[gj] = hv;
            else cluster.map_shared_rank(h0new_local, gd)[u0 + gj] = hv;
        }
        if (XB) {
            __syncthreads();
            send_state(h0new_local, 0);
            xwait(0);
        } else {
            cluster.sync();
        }
        if (trp && tid == 0) trp[4] = clock64();
        // layer 1: the input product continues the sums of the state product made ahead
#pragma unroll
        for (int i = 0; i < NRG; ++i) z[i] = zp1[i];
        rows_dot<NRG>(Wih1, 4 * nu, PH, h0new_local, warp, lane, z);
        rows_reduce<NRG>(z);
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < NRG; ++i) {
                const int r = warp + kGreedyWarps * i;
                if (r < 4 * nu) zrow[r] = z[i] + bias1s[r];
            }
        }
        __syncthreads();
        if (gate_thread) {
            const float zi = zrow[gj * 4], zf = zrow[gj * 4 + 1], zg = zrow[gj * 4 + 2], zo = zrow[gj * 4 + 3];
            c_l1 = sigmoidf_(zf) * c_l1 + sigmoidf_(zi) * tanhf_(zg);
            const __half hv = __float2half_rn(sigmoidf_(zo) * tanhf_(c_l1));
            if (XB) hst[gj] = hv;
            else cluster.map_shared_rank(h1new_local, gd)[u0 + gj] = hv;
        }
        if (XB) {
            __syncthreads();
            send_state(h1new_local, 1);
            xwait(1);
        } else {
            cluster.sync();
        }
        if (trp && tid == 0) trp[5] = clock64();
        // prediction half of the joint: Pj[j] = W1p[j,:] . h1 ; lane d delivers the value to CTA d
        float zj[NRJ];
#pragma unroll
        for (int i = 0; i < NRJ; ++i) zj[i] = 0.f;
        rows_dot<NRJ>(W1p, nj, PH, h1new_local, warp, lane, zj);
        rows_reduce<NRJ>(zj);
        if (lane < C && !(XB && dead)) {
#pragma unroll
            for (int i = 0; i < NRJ; ++i) {
                const int q = warp + kGreedyWarps * i;
                if (q < nj) {
                    if (XB)
                        g_st_async_b32(g_mapa(g_smem_u32(Pj + j0 + q), lane), __float_as_uint(zj[i]),
                                       g_mapa(xbar0 + 8u * (4 + (n_eval & 1u)), lane));
                    else
                        cluster.map_shared_rank(Pj, lane)[j0 + q] = zj[i];
                }
            }
        }
        if (trp && tid == 0) trp[6] = clock64();
        // The state products of the NEXT evaluation depend on no token: they run while the joint values travel (between
        // the arrive and the wait of the cluster barrier in the other variant), and stay in registers, as per-lane
        // partial sums, until that evaluation comes.
        if (!XB) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
#pragma unroll
        for (int i = 0; i < NRG; ++i) zp0[i] = zp1[i] = 0.f;
        rows_dot<NRG>(Whh0, 4 * nu, PH, h0new_local, warp, lane, zp0);
        rows_dot<NRG>(Whh1, 4 * nu, PH, h1new_local, warp, lane, zp1);
        if (XB) xwait(2);
        else asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        ++n_eval;
        if (trp && tid == 0) trp[7] = clock64();
    };

    for (int utt = cluster_id; utt < a.n_utts; utt += n_clusters) {
        const float* E = a.E + (size_t)utt * a.Tp * JH;
        int* tokens = a.tokens + (size_t)utt * a.Tp;
        float* logits = a.logits ? a.logits + (size_t)utt * a.Tp * V : nullptr;
        for (int i = tid; i < 2 * PH; i += nthr) {
            h0buf[i] = __float2half_rn(0.f);
            h1buf[i] = __float2half_rn(0.f);
        }
        c_l0 = 0.f;
        c_l1 = 0.f;
#pragma unroll
        for (int i = 0; i < NRG; ++i) zp0[i] = zp1[i] = 0.f;  // products with the zero state
        cluster.sync();  // staged weights and zeroed states visible; nobody still writes into my buffers
        int e = 0, n_emit = 0;
        float e_next[2] = {0.f, 0.f};  // E[t+1] for z elements tid and tid+nthr
        if (a.Tp > 0) {
            if (tid < JH) e_next[0] = __ldcg(E + tid);
            if (tid + nthr < JH) e_next[1] = __ldcg(E + tid + nthr);
        }
        // iteration -1 is the start of sequence: the blank row of the embedding, zero state (one inlined copy of the
        // evaluation serves both: the loop body is the kernel's instruction footprint)
        for (int t = -1; t < a.Tp; ++t) {
            int tok = a.blank;
            trp = nullptr;
            if (t >= 0) {
                trp = (a.trace && utt == 0 && rank == 0) ? a.trace + (size_t)t * 8 : nullptr;
                if (trp && tid == 0) trp[0] = clock64();
                const float e_cur0 = e_next[0], e_cur1 = e_next[1];
                if (t + 1 < a.Tp) {
                    if (tid < JH) e_next[0] = __ldcg(E + (size_t)(t + 1) * JH + tid);
                    if (tid + nthr < JH) e_next[1] = __ldcg(E + (size_t)(t + 1) * JH + tid + nthr);
                }
                if (tid < JH) zs[tid] = __float2half_rn(fmaxf(e_cur0 + Pj[tid], 0.f));
                if (tid + nthr < JH) zs[tid + nthr] = __float2half_rn(fmaxf(e_cur1 + Pj[tid + nthr], 0.f));
                __syncthreads();
                float zv[NRV];
#pragma unroll
                for (int i = 0; i < NRV; ++i) zv[i] = 0.f;
                rows_dot<NRV>(W2, V, JH, zs, warp, lane, zv);
                rows_reduce<NRV>(zv);
                if (lane == 0) {
#pragma unroll
                    for (int i = 0; i < NRV; ++i) {
                        const int r = warp + kGreedyWarps * i;
                        if (r < V) lg[r] = zv[i] + b2s[r];
                    }
                }
                __syncthreads();
                if (trp && tid == 0) trp[1] = clock64();
                // argmax, first maximum wins; every warp repeats it, so no broadcast is needed
                float bv = -INFINITY;
                int best = 0x7fffffff;
                for (int r = lane; r < V; r += 32) {
                    const float v = lg[r];
                    if (v > bv) { bv = v; best = r; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, best, o);
                    if (ov > bv || (ov == bv && oi < best)) { bv = ov; best = oi; }
                }
                if (rank == 0 && logits && tid < V) logits[(size_t)t * V + tid] = lg[tid];
                if (trp && tid == 0) trp[2] = clock64();
                if (best == a.blank) continue;
                if (rank == 0 && tid == 0) tokens[n_emit] = best;
                ++n_emit;
                tok = best;
            }
            pred_eval(tok, e++);  // commits the pending state and evaluates the new label
        }
        if (rank == 0 && tid == 0) a.n_tokens[utt] = n_emit;
    }
    // after a wait that ran out, a peer's stores may still be on their way to this CTA: let them land
    if (XB && (dead || status_aborted(a.status, a.gen)))
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    cluster.sync();  // no CTA leaves while a peer may still address its shared memory
}

// z[i][m] += W[row_i, :] . h_m for M hidden vectors at once: every weight chunk is loaded once and used M times
template <int NR, int M>
__device__ __forceinline__ void rows_dot_multi(const __half* __restrict__ W, int rows, int K, const __half* const* h,
                                               unsigned live, int warp, int lane, float (*z)[M]) {
    const int K8 = K >> 3;
    for (int c = lane; c < K8; c += 32) {
        uint4 wv[NR];
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int r = min(warp + kGreedyWarps * i, rows - 1);
            wv[i] = reinterpret_cast<const uint4*>(W + (size_t)r * K)[c];
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (live & (1u << m)) {
                float xf[8];
                widen8(reinterpret_cast<const uint4*>(h[m])[c], xf);
#pragma unroll
                for (int i = 0; i < NR; ++i) z[i][m] = dot8f(wv[i], xf, z[i][m]);
            }
        }
    }
}

// The same greedy loop for M utterances per cluster in lock step.  The weights in shared memory, the cluster
// barriers and the phase latencies are shared by the M utterances; each keeps its own prediction-network state,
// emission count and transcript.  An utterance whose frame decided "blank" simply sits out the prediction-network
// evaluation of that frame (the mask is the same in every CTA, because every CTA takes every decision).
template <int NRG, int NRJ, int NRV, int M>
__global__ void __launch_bounds__(kGreedyThreads, 1) rnnt_greedy_multi_kernel(GreedyArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    const int C = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int cluster_id = blockIdx.x / C, n_clusters = gridDim.x / C;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int nthr = kGreedyThreads;
    const int PH = a.PH, JH = a.JH, V = a.V;
    const int UP = (PH + C - 1) / C, u0 = rank * UP, nu = max(0, min(UP, PH - u0));
    const int JP = (JH + C - 1) / C, j0 = rank * JP, nj = max(0, min(JP, JH - j0));

    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned char* sp = smem_raw;
    auto carve = [&](size_t bytes) {
        unsigned char* p = sp;
        sp += (bytes + 15) & ~size_t(15);
        return p;
    };
    __half* h0buf = reinterpret_cast<__half*>(carve((size_t)M * 2 * PH * 2));   // [M][2][PH]
    __half* h1buf = reinterpret_cast<__half*>(carve((size_t)M * 2 * PH * 2));
    float* Pj = reinterpret_cast<float*>(carve((size_t)M * JH * 4));            // [M][JH]
    __half* zs = reinterpret_cast<__half*>(carve((size_t)M * JH * 2));          // [M][JH]
    float* zrow = reinterpret_cast<float*>(carve((size_t)M * 4 * UP * 4));      // [M][4UP]
    float* lg = reinterpret_cast<float*>(carve((size_t)M * (V + 1) * 4));       // [M][V+1]
    float* b2s = reinterpret_cast<float*>(carve((size_t)V * 4));
    float* bias1s = reinterpret_cast<float*>(carve((size_t)4 * UP * 4));
    const size_t slice = (size_t)4 * UP * PH * 2;
    const __half* Whh0 = a.Whh0 + (size_t)u0 * 4 * PH;
    const __half* Wih1 = a.Wih1 + (size_t)u0 * 4 * PH;
    const __half* Whh1 = a.Whh1 + (size_t)u0 * 4 * PH;
    const __half* W1p = a.W1p + (size_t)j0 * PH;
    const __half* W2 = a.W2;
    auto stage = [&](const __half* g, size_t halves, size_t cap_bytes) {
        __half* s = reinterpret_cast<__half*>(carve(cap_bytes));
        const uint4* g4 = reinterpret_cast<const uint4*>(g);
        uint4* s4 = reinterpret_cast<uint4*>(s);
        for (size_t i = tid; i < halves / 8; i += nthr) s4[i] = __ldg(g4 + i);
        return (const __half*)s;
    };
    if (a.smem_mask & 1) Whh0 = stage(Whh0, (size_t)4 * nu * PH, slice);
    if (a.smem_mask & 2) Wih1 = stage(Wih1, (size_t)4 * nu * PH, slice);
    if (a.smem_mask & 4) Whh1 = stage(Whh1, (size_t)4 * nu * PH, slice);
    if (a.smem_mask & 8) W1p = stage(W1p, (size_t)nj * PH, (size_t)JP * PH * 2);
    if (a.smem_mask & 16) W2 = stage(W2, (size_t)V * JH, (size_t)V * JH * 2);
    for (int i = tid; i < V; i += nthr) b2s[i] = a.b2[i];
    for (int i = tid; i < 4 * nu; i += nthr) bias1s[i] = a.bias1[(size_t)u0 * 4 + i];

    // gate threads: pair p = (unit j, utterance m), p < nu*M, replicated REP times; replica r writes to CTAs r, r+REP, ...
    const int NG = nu * M;
    const int REP = NG > 0 ? min(C, nthr / NG) : 1;
    const int gp = tid % max(NG, 1), grep = tid / max(NG, 1);
    const bool gate_thread = NG > 0 && grep < REP;
    const int gj = gp / M, gm = gp - gj * M;
    float c_l0 = 0.f, c_l1 = 0.f;

    const int n_groups = (a.n_utts + M - 1) / M;
    for (int grp = cluster_id; grp < n_groups; grp += n_clusters) {
        const int utt0 = grp * M;
        unsigned valid = 0;
        for (int m = 0; m < M; ++m)
            if (utt0 + m < a.n_utts) valid |= 1u << m;
        for (int i = tid; i < M * 2 * PH; i += nthr) {
            h0buf[i] = __float2half_rn(0.f);
            h1buf[i] = __float2half_rn(0.f);
        }
        c_l0 = 0.f;
        c_l1 = 0.f;
        cluster.sync();
        int e[M], n_emit[M], tok[M];
#pragma unroll
        for (int m = 0; m < M; ++m) { e[m] = 0; n_emit[m] = 0; tok[m] = a.blank; }

        // prediction-network evaluation of the utterances in `mask`
        auto pred_eval = [&](unsigned mask) {
            const __half* hp[M];
            float z[NRG][M];
            // layer 0
#pragma unroll
            for (int m = 0; m < M; ++m) hp[m] = h0buf + ((size_t)m * 2 + ((e[m] + 1) & 1)) * PH;
#pragma unroll
            for (int i = 0; i < NRG; ++i)
#pragma unroll
                for (int m = 0; m < M; ++m) z[i][m] = 0.f;
            rows_dot_multi<NRG, M>(Whh0, 4 * nu, PH, hp, mask, warp, lane, z);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int i = 0; i < NRG; ++i)
#pragma unroll
                    for (int m = 0; m < M; ++m) z[i][m] += __shfl_xor_sync(0xffffffffu, z[i][m], o);
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < NRG; ++i) {
                    const int r = warp + kGreedyWarps * i;
                    if (r < 4 * nu) {
#pragma unroll
                        for (int m = 0; m < M; ++m)
                            if (mask & (1u << m))
                                zrow[m * 4 * UP + r] = z[i][m] + __ldg(a.P0 + (size_t)tok[m] * 4 * PH + (size_t)u0 * 4 + r);
                    }
                }
            }
            __syncthreads();
            if (gate_thread && (mask & (1u << gm))) {
                const float* zr = zrow + gm * 4 * UP + gj * 4;
                c_l0 = sigmoidf_(zr[1]) * c_l0 + sigmoidf_(zr[0]) * tanhf_(zr[2]);
                const __half hh = __float2half_rn(sigmoidf_(zr[3]) * tanhf_(c_l0));
                __half* dstl = h0buf + ((size_t)gm * 2 + (e[gm] & 1)) * PH + u0 + gj;
                for (int d = grep; d < C; d += REP) *cluster.map_shared_rank(dstl, d) = hh;
            }
            cluster.sync();
            // layer 1
#pragma unroll
            for (int i = 0; i < NRG; ++i)
#pragma unroll
                for (int m = 0; m < M; ++m) z[i][m] = 0.f;
#pragma unroll
            // state product first, input product second: the summation order of the one-utterance kernel
            for (int m = 0; m < M; ++m) hp[m] = h1buf + ((size_t)m * 2 + ((e[m] + 1) & 1)) * PH;
            rows_dot_multi<NRG, M>(Whh1, 4 * nu, PH, hp, mask, warp, lane, z);
#pragma unroll
            for (int m = 0; m < M; ++m) hp[m] = h0buf + ((size_t)m * 2 + (e[m] & 1)) * PH;
            rows_dot_multi<NRG, M>(Wih1, 4 * nu, PH, hp, mask, warp, lane, z);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int i = 0; i < NRG; ++i)
#pragma unroll
                    for (int m = 0; m < M; ++m) z[i][m] += __shfl_xor_sync(0xffffffffu, z[i][m], o);
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < NRG; ++i) {
                    const int r = warp + kGreedyWarps * i;
                    if (r < 4 * nu) {
#pragma unroll
                        for (int m = 0; m < M; ++m)
                            if (mask & (1u << m)) zrow[m * 4 * UP + r] = z[i][m] + bias1s[r];
                    }
                }
            }
            __syncthreads();
            if (gate_thread && (mask & (1u << gm))) {
                const float* zr = zrow + gm * 4 * UP + gj * 4;
                c_l1 = sigmoidf_(zr[1]) * c_l1 + sigmoidf_(zr[0]) * tanhf_(zr[2]);
                const __half hh = __float2half_rn(sigmoidf_(zr[3]) * tanhf_(c_l1));
                __half* dstl = h1buf + ((size_t)gm * 2 + (e[gm] & 1)) * PH + u0 + gj;
                for (int d = grep; d < C; d += REP) *cluster.map_shared_rank(dstl, d) = hh;
            }
            cluster.sync();
            // prediction half of the joint
            float zj[NRJ][M];
#pragma unroll
            for (int i = 0; i < NRJ; ++i)
#pragma unroll
                for (int m = 0; m < M; ++m) zj[i][m] = 0.f;
#pragma unroll
            for (int m = 0; m < M; ++m) hp[m] = h1buf + ((size_t)m * 2 + (e[m] & 1)) * PH;
            rows_dot_multi<NRJ, M>(W1p, nj, PH, hp, mask, warp, lane, zj);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int i = 0; i < NRJ; ++i)
#pragma unroll
                    for (int m = 0; m < M; ++m) zj[i][m] += __shfl_xor_sync(0xffffffffu, zj[i][m], o);
            if (lane < C) {
#pragma unroll
                for (int i = 0; i < NRJ; ++i) {
                    const int q = warp + kGreedyWarps * i;
                    if (q < nj) {
#pragma unroll
                        for (int m = 0; m < M; ++m)
                            if (mask & (1u << m)) cluster.map_shared_rank(Pj + (size_t)m * JH, lane)[j0 + q] = zj[i][m];
                    }
                }
            }
            cluster.sync();
#pragma unroll
            for (int m = 0; m < M; ++m)
                if (mask & (1u << m)) ++e[m];
        };

        pred_eval(valid);  // start of sequence for every utterance of the group
        for (int t = 0; t < a.Tp; ++t) {
            // joint: z_m = relu(E_m[t] + Pj_m)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                if (valid & (1u << m)) {
                    const float* E = a.E + ((size_t)(utt0 + m) * a.Tp + t) * JH;
                    for (int i = tid; i < JH; i += nthr)
                        zs[m * JH + i] = __float2half_rn(fmaxf(__ldcg(E + i) + Pj[m * JH + i], 0.f));
                }
            }
            __syncthreads();
            float zv[NRV][M];
#pragma unroll
            for (int i = 0; i < NRV; ++i)
#pragma unroll
                for (int m = 0; m < M; ++m) zv[i][m] = 0.f;
            const __half* zp[M];
#pragma unroll
            for (int m = 0; m < M; ++m) zp[m] = zs + (size_t)m * JH;
            rows_dot_multi<NRV, M>(W2, V, JH, zp, valid, warp, lane, zv);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int i = 0; i < NRV; ++i)
#pragma unroll
                    for (int m = 0; m < M; ++m) zv[i][m] += __shfl_xor_sync(0xffffffffu, zv[i][m], o);
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < NRV; ++i) {
                    const int r = warp + kGreedyWarps * i;
                    if (r < V) {
#pragma unroll
                        for (int m = 0; m < M; ++m) lg[m * (V + 1) + r] = zv[i][m] + b2s[r];
                    }
                }
            }
            __syncthreads();
            unsigned emit = 0;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                if (!(valid & (1u << m))) continue;
                float bv = -INFINITY;
                int best = 0x7fffffff;
                for (int r = lane; r < V; r += 32) {
                    const float v = lg[m * (V + 1) + r];
                    if (v > bv) { bv = v; best = r; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, best, o);
                    if (ov > bv || (ov == bv && oi < best)) { bv = ov; best = oi; }
                }
                if (rank == 0 && a.logits && tid < V)
                    a.logits[((size_t)(utt0 + m) * a.Tp + t) * V + tid] = lg[m * (V + 1) + tid];
                if (best != a.blank) {
                    if (rank == 0 && tid == 0) a.tokens[(size_t)(utt0 + m) * a.Tp + n_emit[m]] = best;
                    ++n_emit[m];
                    tok[m] = best;
                    emit |= 1u << m;
                }
            }
            if (emit) pred_eval(emit);
            else __syncthreads();  // zs / lg are rewritten next frame
        }
        if (rank == 0 && tid == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m)
                if (valid & (1u << m)) a.n_tokens[utt0 + m] = n_emit[m];
        }
    }
    cluster.sync();
}

// ---------------------------------------------------------------------------------------------
// Tensor-core variant of the greedy loop: 8 utterances per cluster, one column of an m16n8k16 tile each.
// Every matrix-vector product of the loop becomes [rows x K] . [K x 8]; the weights sit in shared memory as
// ldmatrix operands (16-byte chunks XOR-swizzled by row, no padding), the hidden vectors are the B operand.
// Needs: 4*ceil(PH/C) and ceil(JH/C) multiples of 16, PH and JH multiples of 64, V <= 32.
// ---------------------------------------------------------------------------------------------
constexpr int kMmaUtts = 8;

__device__ __forceinline__ void g_ldmatrix_x4(uint32_t* r, const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void g_mma_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// element (r, k) of a swizzled [rows x K] matrix in shared memory (K % 64 == 0)
__device__ __forceinline__ const __half* swz(const __half* base, int r, int k, int K) {
    return base + (size_t)r * K + ((((k >> 3) ^ (r & 7)) << 3) | (k & 7));
}
__device__ __forceinline__ void stage_swizzled(__half* dst, const __half* src, int rows_valid, int rows_total, int K,
                                               int tid, int nthr) {
    const int K8 = K >> 3;
    for (int i = tid; i < rows_total * K8; i += nthr) {
        const int r = i / K8, c = i - r * K8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows_valid) v = __ldg(reinterpret_cast<const uint4*>(src + (size_t)r * K) + c);
        *reinterpret_cast<uint4*>(dst + (size_t)r * K + ((c ^ (r & 7)) << 3)) = v;
    }
}
// acc += A[mt*16 .. +16, kt0*16 .. (kt0+nkt)*16) . B, A swizzled in shared memory, B = hb[n][k] with row pitch `bp`
// (splitting the k-tiles over independent accumulators was measured and does not shorten these short chains)
// NKT > 0: the number of k-tiles is known at compile time (and so should K and bp be: the loop unrolls fully and the
// addresses fold); NKT == 0: run-time count `nkt`.
template <int NKT>
__device__ __forceinline__ void mma_rows_smem(float* acc, const __half* A, int K, int mt, int kt0, int nkt,
                                              const __half* hb, int bp, int lane) {
    const int a_row = mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int a_col = (lane >> 4) * 8;
    const __half* brow = hb + (size_t)(lane >> 2) * bp + (lane & 3) * 2;
    if constexpr (NKT > 0) {
        const __half* arow = A + (size_t)a_row * K;
        const int c0 = 2 * kt0 + (lane >> 4), r7 = a_row & 7;
        brow += kt0 << 4;
        // two chains of dependent tile products instead of one: odd k-tiles go to a second accumulator
        float acc_odd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < NKT; ++i) {
            uint32_t af[4];
            g_ldmatrix_x4(af, arow + (((c0 + 2 * i) ^ r7) << 3));
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + 16 * i);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + 16 * i + 8);
            g_mma_16816((i & 1) ? acc_odd : acc, af, b0, b1);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += acc_odd[q];
    } else {
#pragma unroll 4
        for (int kt = kt0; kt < kt0 + nkt; ++kt) {
            const int k0 = kt << 4;
            uint32_t af[4];
            g_ldmatrix_x4(af, swz(A, a_row, k0 + a_col, K));
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + k0);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + k0 + 8);
            g_mma_16816(acc, af, b0, b1);
        }
    }
}
// same with A read straight from global memory (row-major, pitch K) through L1
template <int NKT>
__device__ __forceinline__ void mma_rows_gmem(float* acc, const __half* A, int K, int mt, int kt0, int nkt,
                                              const __half* hb, int bp, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const __half* a_lo = A + (size_t)(mt * 16 + g) * K + 2 * t;
    const __half* a_hi = a_lo + (size_t)8 * K;
    const __half* brow = hb + (size_t)g * bp + 2 * t;
    if constexpr (NKT > 0) {
        // every fragment of the product is requested before the first multiply: one trip to L1 / L2, not NKT of them
        uint32_t af[NKT][4];
        a_lo += kt0 << 4; a_hi += kt0 << 4; brow += kt0 << 4;
#pragma unroll
        for (int i = 0; i < NKT; ++i) {
            af[i][0] = __ldg(reinterpret_cast<const uint32_t*>(a_lo + 16 * i));
            af[i][1] = __ldg(reinterpret_cast<const uint32_t*>(a_hi + 16 * i));
            af[i][2] = __ldg(reinterpret_cast<const uint32_t*>(a_lo + 16 * i + 8));
            af[i][3] = __ldg(reinterpret_cast<const uint32_t*>(a_hi + 16 * i + 8));
        }
#pragma unroll
        for (int i = 0; i < NKT; ++i) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + 16 * i);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + 16 * i + 8);
            g_mma_16816(acc, af[i], b0, b1);
        }
    } else {
#pragma unroll 5
        for (int kt = kt0; kt < kt0 + nkt; ++kt) {
            const int k0 = kt << 4;
            uint32_t af[4];
            af[0] = __ldg(reinterpret_cast<const uint32_t*>(a_lo + k0));
            af[1] = __ldg(reinterpret_cast<const uint32_t*>(a_hi + k0));
            af[2] = __ldg(reinterpret_cast<const uint32_t*>(a_lo + k0 + 8));
            af[3] = __ldg(reinterpret_cast<const uint32_t*>(a_hi + k0 + 8));
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + k0);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + k0 + 8);
            g_mma_16816(acc, af, b0, b1);
        }
    }
}
// the same product with the A fragments already in registers
template <int NKT>
__device__ __forceinline__ void frags_mma(float* acc, const uint4* af, int kt0, const __half* hb, int bp, int lane) {
    const __half* brow = hb + (size_t)(lane >> 2) * bp + (lane & 3) * 2 + (kt0 << 4);
#pragma unroll
    for (int i = 0; i < NKT; ++i) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow + 16 * i);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + 16 * i + 8);
        const uint32_t a4[4] = {af[i].x, af[i].y, af[i].z, af[i].w};
        g_mma_16816(acc, a4, b0, b1);
    }
}
// accumulator tile -> part[split][n][row] (fp32): thread holds (row g, cols 2t,2t+1) and (row g+8, same cols)
__device__ __forceinline__ void store_acc(float* part, int ld, int mt, const float* acc, int lane) {
    const int g = lane >> 2, t = lane & 3;
    part[(size_t)(2 * t) * ld + mt * 16 + g] = acc[0];
    part[(size_t)(2 * t + 1) * ld + mt * 16 + g] = acc[1];
    part[(size_t)(2 * t) * ld + mt * 16 + g + 8] = acc[2];
    part[(size_t)(2 * t + 1) * ld + mt * 16 + g + 8] = acc[3];
}

// PHC / JHC: pred_hidden and joint_hidden as compile-time constants (0 = taken from the arguments); with them every
// product loop has a constant trip count and constant strides.
template <int PHC, int JHC>
__global__ void __launch_bounds__(kGreedyThreads, 1) rnnt_greedy_mma_kernel(GreedyArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    const int C = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int cluster_id = blockIdx.x / C, n_clusters = gridDim.x / C;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int nthr = kGreedyThreads;
    constexpr int M = kMmaUtts;
    const int PH = PHC > 0 ? PHC : a.PH, JH = JHC > 0 ? JHC : a.JH, V = a.V;
    // constant trip counts of the product loops (0 = run time): half of K for the gate products, all of K for the
    // state product under the exchange, a quarter of K for the joint half, a quarter of JH for the logits
    constexpr int NK_HALF = (PHC > 0 && PHC % 32 == 0) ? PHC / 32 : 0;
    constexpr int NK_FULL = NK_HALF > 0 ? PHC / 16 : 0;
    constexpr int NK_PJ = (PHC > 0 && PHC % 64 == 0) ? PHC / 64 : 0;
    constexpr int NK_LG = (JHC > 0 && JHC % 64 == 0) ? JHC / 64 : 0;
    const int UP = PH / C, u0 = rank * UP, RG = 4 * UP;      // gate rows of this CTA (multiple of 16)
    const int JP = JH / C, j0 = rank * JP;                  // joint rows of this CTA (multiple of 16)
    const int hp = PH + 8, zp = JH + 8;                      // pitches of the B-operand buffers
    const int MTG = RG / 16, MTJ = JP / 16, KTP = PH / 16, KTJ = JH / 16;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    unsigned char* sp = smem_raw;
    auto carve = [&](size_t bytes) {
        unsigned char* p = sp;
        sp += (bytes + 15) & ~size_t(15);
        return p;
    };
    __half* Whh0 = reinterpret_cast<__half*>(carve((size_t)RG * PH * 2));
    __half* Wih1 = reinterpret_cast<__half*>(carve((size_t)RG * PH * 2));
    __half* Whh1 = reinterpret_cast<__half*>(carve((size_t)RG * PH * 2));
    __half* W2s = reinterpret_cast<__half*>(carve((size_t)32 * JH * 2));
    __half* h0buf = reinterpret_cast<__half*>(carve((size_t)2 * M * hp * 2));   // [2][M][hp]
    __half* h1buf = reinterpret_cast<__half*>(carve((size_t)2 * M * hp * 2));
    __half* Pj = reinterpret_cast<__half*>(carve((size_t)M * JH * 2));           // [M][JH]
    __half* zs = reinterpret_cast<__half*>(carve((size_t)M * zp * 2));           // [M][zp]
    // partial sums: [2 splits][M][RG] for the gate phases, [4 splits][M][32] for the joint / logits phases
    const int part_floats = 2 * M * RG > 4 * M * 32 ? 2 * M * RG : 4 * M * 32;
    float* part = reinterpret_cast<float*>(carve((size_t)part_floats * 4));
    const int gl = RG, jl = 32;   // row pitches of the two uses
    // staging of this CTA's new values before they go to the other CTAs as 8- / 16-byte stores
    __half* stage = reinterpret_cast<__half*>(carve((size_t)M * 32 * 4));        // [M][UP] or [M][JP] halves
    float* b2s = reinterpret_cast<float*>(carve((size_t)32 * 4));
    float* bias1s = reinterpret_cast<float*>(carve((size_t)RG * 4));
    int* best_s = reinterpret_cast<int*>(carve((size_t)M * 4));
    // exchange barriers [exchange 0..2 = layer-0 state, layer-1 state, joint half][use & 1]
    const uint32_t xbar0 = g_smem_u32(carve(6 * 8));
    const __half* W1p = a.W1p + (size_t)j0 * PH;  // read through L1: no room left in shared memory
    if (tid == 0) {
        for (int i = 0; i < 6; ++i) g_xbar_init(xbar0 + 8u * i);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    uint32_t n_eval = 0;    // evaluations so far: use n_eval of every exchange takes barrier n_eval & 1, phase n_eval >> 1
    bool dead = false;      // a wait of this thread ran out: no more waits, no more sends
    auto xwait = [&](int x) {
        if (dead) return;
        if (!g_xbar_wait(xbar0 + 8u * (2 * x + (n_eval & 1u)), (n_eval >> 1) & 1u, a.status, a.gen, a.poll_limit)) {
            dead = true;
            status_raise(a.status, a.gen, PIMB200_ERR_TIMEOUT);
        }
    };

    stage_swizzled(Whh0, a.Whh0 + (size_t)u0 * 4 * PH, RG, RG, PH, tid, nthr);
    stage_swizzled(Wih1, a.Wih1 + (size_t)u0 * 4 * PH, RG, RG, PH, tid, nthr);
    stage_swizzled(Whh1, a.Whh1 + (size_t)u0 * 4 * PH, RG, RG, PH, tid, nthr);
    stage_swizzled(W2s, a.W2, V, 32, JH, tid, nthr);
    for (int i = tid; i < 32; i += nthr) b2s[i] = i < V ? a.b2[i] : -INFINITY;
    for (int i = tid; i < RG; i += nthr) bias1s[i] = a.bias1[(size_t)u0 * 4 + i];

    // gate threads: thread p < UP*M owns (unit gj, utterance gn)
    const int NG = UP * M;
    const bool gate_thread = tid < NG;
    const int gj = gate_thread ? tid / M : 0, gn = gate_thread ? tid - gj * M : 0;
    float c_l0 = 0.f, c_l1 = 0.f;
    // warp roles of the gate-phase products: role 0 / 1 = the two K halves, role 2 = the product with the state of the
    // previous evaluation (independent of the exchange in flight)
    const int mt_w = warp % MTG, role = warp / MTG;
    const int k_half = KTP / 2;
    // joint-phase roles: m-tile and K quarter
    const int mtj_w = warp % MTJ, kqj = warp / MTJ;
    const int perj = (KTP + 3) / 4;
    // items of the two all-to-all copies, fixed per thread: (destination CTA d, utterance n, chunk c)
    const int CH = UP / 4, CJ = JP / 8;                     // 8-byte chunks of a state row, 16-byte chunks of a joint row
    const int n_hitems = C * M * CH, n_jitems = C * M * CJ;
    int h_item[2], j_item;                                  // packed d << 16 | n << 8 | c, or -1
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int i = tid + q * nthr;
        h_item[q] = -1;
        if (i < n_hitems) {
            const int d = i / (M * CH), r = i - d * (M * CH), n = r / CH, c = r - n * CH;
            h_item[q] = (d << 16) | (n << 8) | c;
        }
    }
    j_item = -1;
    if (tid < n_jitems) {
        const int d = tid / (M * CJ), r = tid - d * (M * CJ), n = r / CJ, c = r - n * CJ;
        j_item = (d << 16) | (n << 8) | c;
    }

    const int n_groups = (a.n_utts + M - 1) / M;
    for (int grp = cluster_id; grp < n_groups; grp += n_clusters) {
        const int utt0 = grp * M;
        unsigned valid = 0;
        for (int m = 0; m < M; ++m)
            if (utt0 + m < a.n_utts) valid |= 1u << m;
        for (int i = tid; i < 2 * M * hp; i += nthr) {
            h0buf[i] = __float2half_rn(0.f);
            h1buf[i] = __float2half_rn(0.f);
        }
        for (int i = tid; i < M * zp; i += nthr) zs[i] = __float2half_rn(0.f);
        for (int i = tid; i < M * JH; i += nthr) Pj[i] = __float2half_rn(0.f);
        if (tid < M) best_s[tid] = a.blank;   // the start-of-sequence evaluation embeds the blank symbol
        c_l0 = 0.f;
        c_l1 = 0.f;
        cluster.sync();
        // all utterances of a group evaluate the prediction network the same number of times only if they emit in
        // the same frames; each keeps its own parity, packed one bit per utterance
        unsigned par = 0;          // bit n = parity of utterance n's next evaluation
        int n_emit[M];
#pragma unroll
        for (int m = 0; m < M; ++m) n_emit[m] = 0;

        // Because an m16n8k16 pass always covers all 8 columns, the B operand of an evaluation must hold, for every
        // column, the state that utterance will read: buffers are indexed [parity][n], and a column that sits the
        // evaluation out simply produces a value nobody stores.
        long long* trp = nullptr;
        float acc_l0[4] = {0.f, 0.f, 0.f, 0.f};   // Whh0 . h0 of the coming evaluation (zero state at the start)
        // new state values of this CTA (stage[n][0..UP)) -> plane (par>>n)&1 of `buf` in every CTA, 8 bytes a store
        auto scatter_state = [&](__half* buf, unsigned mask, int x) {
            const uint32_t bar = xbar0 + 8u * (2 * x + (n_eval & 1u));
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int it = h_item[q];
                if (it >= 0 && !dead) {
                    const int d = it >> 16, n = (it >> 8) & 0xff, c = it & 0xff;
                    if (mask & (1u << n)) {
                        const uint2 v = *reinterpret_cast<const uint2*>(stage + n * UP + c * 4);
                        __half* dstl = buf + ((size_t)((par >> n) & 1u) * M + n) * hp + u0 + c * 4;
                        g_st_async_v2(g_mapa(g_smem_u32(dstl), d), v, g_mapa(bar, d));
                    }
                }
            }
        };
        auto pred_eval = [&](unsigned mask) {
            const bool mine = gate_thread && (mask & (1u << gn));
            if (tid == 0) {   // what this CTA will receive in the three exchanges of this evaluation
                const uint32_t nm = (uint32_t)__popc(mask), b = n_eval & 1u;
                g_xbar_expect(xbar0 + 8u * b, nm * PH * 2);
                g_xbar_expect(xbar0 + 8u * (2 + b), nm * PH * 2);
                g_xbar_expect(xbar0 + 8u * (4 + b), nm * JH * 2);
            }
            // input term of layer 0 for the symbol just emitted: fetched now, used after the first product
            float4 p0v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (mine) p0v = __ldg(reinterpret_cast<const float4*>(a.P0 + (size_t)best_s[gn] * 4 * PH + (size_t)(u0 + gj) * 4));
            // ---- layer 0: z = Whh0 . h0prev (+ P0[tok]); the two K halves of the product were made by roles 0 and 1
            //      during the previous evaluation (acc_l0), while its layer-1 state travelled
            float acc2[4] = {0.f, 0.f, 0.f, 0.f};
            if (role < 2) store_acc(part + (size_t)role * M * gl, gl, mt_w, acc_l0, lane);
            __syncthreads();
            if (trp && tid == 0) trp[4] = clock64();
            if (mine) {
                const float4 za = *reinterpret_cast<const float4*>(part + (size_t)gn * gl + gj * 4);
                const float4 zb = *reinterpret_cast<const float4*>(part + (size_t)(M + gn) * gl + gj * 4);
                const float zi = za.x + zb.x + p0v.x, zf = za.y + zb.y + p0v.y, zg = za.z + zb.z + p0v.z,
                            zo = za.w + zb.w + p0v.w;
                c_l0 = sigmoidf_(zf) * c_l0 + sigmoidf_(zi) * tanhf_(zg);
                stage[gn * UP + gj] = __float2half_rn(sigmoidf_(zo) * tanhf_(c_l0));
            }
            __syncthreads();
            scatter_state(h0buf, mask, 0);
            // the state product of layer 1 does not depend on the exchange in flight: roles 0 and 2 make its two K halves
            // while the values travel, and continue the same sums with the input product afterwards
            if (role == 0 || role == 2) {
                const int n = lane >> 2;
                const unsigned pn = (par >> n) & 1u;   // column n reads the plane written by its previous evaluation
                mma_rows_smem<NK_HALF>(acc2, Whh1, PH, mt_w, role ? k_half : 0, role ? KTP - k_half : k_half,
                                       h1buf + (size_t)((pn ^ 1u) * M) * hp, hp, lane);
            }
            xwait(0);
            if (trp && tid == 0) trp[5] = clock64();
            // ---- layer 1: z = Wih1 . h0new + Whh1 . h1prev + bias: role 0 adds the first K half of the input product to
            //      the half it holds, role 2 the second
            if (role == 0 || role == 2) {
                const int n = lane >> 2;
                const unsigned pn = (par >> n) & 1u;
                const __half* hb = h0buf + (size_t)(pn * M) * hp;
                mma_rows_smem<NK_HALF>(acc2, Wih1, PH, mt_w, role ? k_half : 0, role ? KTP - k_half : k_half, hb, hp, lane);
                store_acc(part + (size_t)(role ? M : 0) * gl, gl, mt_w, acc2, lane);
            }
            __syncthreads();
            if (mine) {
                const float4 za = *reinterpret_cast<const float4*>(part + (size_t)gn * gl + gj * 4);
                const float4 zb = *reinterpret_cast<const float4*>(part + (size_t)(M + gn) * gl + gj * 4);
                const float4 bb = *reinterpret_cast<const float4*>(bias1s + gj * 4);
                const float zi = za.x + zb.x + bb.x, zf = za.y + zb.y + bb.y, zg = za.z + zb.z + bb.z,
                            zo = za.w + zb.w + bb.w;
                c_l1 = sigmoidf_(zf) * c_l1 + sigmoidf_(zi) * tanhf_(zg);
                stage[gn * UP + gj] = __float2half_rn(sigmoidf_(zo) * tanhf_(c_l1));
            }
            __syncthreads();
            scatter_state(h1buf, mask, 1);
            // while the layer-1 state travels: the layer-0 state product of the NEXT evaluation.  It depends on no
            // symbol, and column n will read the plane its latest evaluation wrote, which for the columns of this
            // evaluation is the one received above.
            if (role < 2) {
                const int n = lane >> 2;
                const unsigned pl = (((par ^ mask) >> n) & 1u) ^ 1u;
#pragma unroll
                for (int q = 0; q < 4; ++q) acc_l0[q] = 0.f;
                mma_rows_smem<NK_HALF>(acc_l0, Whh0, PH, mt_w, role ? k_half : 0, role ? KTP - k_half : k_half,
                                       h0buf + (size_t)(pl * M) * hp, hp, lane);
            }
            // the weights of the joint half come from global memory (L1 / L2), in fragment order when the sizes are
            // compiled in: one 16-byte load per k-tile and lane, asked for now and multiplied after the wait
            uint4 wj[NK_PJ > 0 ? NK_PJ : 1];
            const bool frag = NK_PJ > 0 && a.W1pf != nullptr;
            if (frag && warp < 4 * MTJ) {
                const uint4* fp = a.W1pf + ((((size_t)rank * MTJ + mtj_w) * 4 + kqj) * NK_PJ) * 32 + lane;
#pragma unroll
                for (int i = 0; i < NK_PJ; ++i) wj[i] = __ldg(fp + i * 32);
            }
            xwait(1);
            if (trp && tid == 0) trp[6] = clock64();
            // ---- prediction half of the joint: Pj[n][j0 + q] = W1p[q,:] . h1new[n]; four K quarters per m-tile
            if (warp < 4 * MTJ) {
                const int k_lo = kqj * perj, k_n = max(0, min(perj, KTP - k_lo));
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const int n = lane >> 2;
                const __half* hb = h1buf + (size_t)(((par >> n) & 1u) * M) * hp;
                if (frag) frags_mma<NK_PJ>(acc, wj, k_lo, hb, hp, lane);
                else mma_rows_gmem<NK_PJ>(acc, W1p, PH, mtj_w, k_lo, k_n, hb, hp, lane);
                store_acc(part + (size_t)kqj * M * jl, jl, mtj_w, acc, lane);
            }
            __syncthreads();
            if (tid < M * 32) {   // (utterance n, joint row q of this CTA's slice)
                const int n = tid >> 5, q = tid & 31;
                if (q < JP) {
                    const float sum = (part[(size_t)n * jl + q] + part[(size_t)(M + n) * jl + q]) +
                                      (part[(size_t)(2 * M + n) * jl + q] + part[(size_t)(3 * M + n) * jl + q]);
                    stage[n * JP + q] = __float2half_rn(sum);
                }
            }
            __syncthreads();
            if (j_item >= 0) {
                const int d = j_item >> 16, n = (j_item >> 8) & 0xff, c = j_item & 0xff;
                if ((mask & (1u << n)) && !dead) {
                    const uint4 v = *reinterpret_cast<const uint4*>(stage + n * JP + c * 8);
                    g_st_async_v4(g_mapa(g_smem_u32(Pj + (size_t)n * JH + j0 + c * 8), d), v,
                                  g_mapa(xbar0 + 8u * (4 + (n_eval & 1u)), d));
                }
            }
            xwait(2);
            if (trp && tid == 0) trp[7] = clock64();
            par ^= mask;
            ++n_eval;
        };

        // E of the next frame is fetched one frame ahead (its L2 latency would otherwise open every frame)
        // When JH equals the block size (the benchmark's 512) a thread owns 8 consecutive columns of one utterance: two
        // 16-byte loads of E, one of Pj and one 16-byte store of z per frame, and no division in the frame loop.
        const bool square = (JH == nthr) && (M == 8);
        const int zn = tid >> 6, zk = (tid & 63) * 8;      // (utterance, first column) of this thread in that case
        const bool zlive = (valid >> zn) & 1u;
        float4 e_lo = make_float4(0.f, 0.f, 0.f, 0.f), e_hi = e_lo;
        auto load_E = [&](int t) {
            if (zlive && t < a.Tp) {
                const float4* ep = reinterpret_cast<const float4*>(a.E + ((size_t)(utt0 + zn) * a.Tp + t) * JH + zk);
                e_lo = __ldcg(ep);
                e_hi = __ldcg(ep + 1);
                // E streams from HBM once; pull the rows of the frames after this one into L2 now, so that their loads
                // (which the scheduler makes other phases wait for) return with L2 latency
                if (t + 2 < a.Tp) asm volatile("prefetch.global.L2 [%0];" ::"l"(ep + (size_t)2 * (JH / 4)));
                if (t + 1 < a.Tp && t == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(ep + (size_t)(JH / 4)));
            }
        };
        if (square) load_E(0);
        // iteration -1 is the start of sequence: every utterance evaluates the blank symbol from the zero state (one
        // inlined copy of the evaluation serves both: the loop body is the kernel's instruction footprint)
        for (int t = -1; t < a.Tp; ++t) {
            unsigned emit = valid;
            trp = nullptr;
            if (t >= 0) {
                trp = (a.trace && grp == 0 && rank == 0) ? a.trace + (size_t)t * 8 : nullptr;
                if (trp && tid == 0) trp[0] = clock64();
                // ---- joint input z[n] = relu(E[n][t] + Pj[n]) in fp16
                if (square) {
                    if (zlive) {
                        const uint4 pj = *reinterpret_cast<const uint4*>(Pj + (size_t)zn * JH + zk);
                        const float2 p0 = h2f2(pj.x), p1 = h2f2(pj.y), p2 = h2f2(pj.z), p3 = h2f2(pj.w);
                        uint4 out;
                        __half2 h;
                        h = __floats2half2_rn(fmaxf(e_lo.x + p0.x, 0.f), fmaxf(e_lo.y + p0.y, 0.f)); out.x = *reinterpret_cast<uint32_t*>(&h);
                        h = __floats2half2_rn(fmaxf(e_lo.z + p1.x, 0.f), fmaxf(e_lo.w + p1.y, 0.f)); out.y = *reinterpret_cast<uint32_t*>(&h);
                        h = __floats2half2_rn(fmaxf(e_hi.x + p2.x, 0.f), fmaxf(e_hi.y + p2.y, 0.f)); out.z = *reinterpret_cast<uint32_t*>(&h);
                        h = __floats2half2_rn(fmaxf(e_hi.z + p3.x, 0.f), fmaxf(e_hi.w + p3.y, 0.f)); out.w = *reinterpret_cast<uint32_t*>(&h);
                        *reinterpret_cast<uint4*>(zs + (size_t)zn * zp + zk) = out;
                    }
                    load_E(t + 1);
                } else {
                    for (int i = tid; i < M * JH; i += nthr) {
                        const int n = i / JH, k = i - n * JH;
                        if (valid & (1u << n)) {
                            const float e = __ldcg(a.E + ((size_t)(utt0 + n) * a.Tp + t) * JH + k);
                            zs[(size_t)n * zp + k] = __float2half_rn(fmaxf(e + __half2float(Pj[i]), 0.f));
                        }
                    }
                }
                __syncthreads();
                if (trp && tid == 0) trp[1] = clock64();
                // ---- logits[n][r] = W2[r,:] . z[n] + b2[r]: 2 m-tiles x 4 K quarters
                if (warp < 8) {
                    const int mt = warp & 1, kq = warp >> 1;
                    const int per = (KTJ + 3) / 4, k_lo = kq * per, k_n = max(0, min(per, KTJ - k_lo));
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_rows_smem<NK_LG>(acc, W2s, JH, mt, k_lo, k_n, zs, zp, lane);
                    store_acc(part + (size_t)kq * M * jl, jl, mt, acc, lane);
                }
                __syncthreads();
                if (trp && tid == 0) trp[2] = clock64();
                if (tid < M * 32) {
                    const int n = tid >> 5, r = tid & 31;   // warp n handles utterance n, lane = vocabulary row
                    float v = (part[(size_t)n * jl + r] + part[(size_t)(M + n) * jl + r]) +
                              (part[(size_t)(2 * M + n) * jl + r] + part[(size_t)(3 * M + n) * jl + r]) + b2s[r];
                    // arg max over the 32 lanes, lowest index on ties: two warp reductions on an order-preserving integer
                    // image of the value (ten dependent shuffles measured ~2.6 k cycles here)
                    uint32_t key = __float_as_uint(v);
                    key = (key & 0x80000000u) ? ~key : (key | 0x80000000u);
                    const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
                    const int best = (int)__reduce_min_sync(0xffffffffu, key == kmax ? (uint32_t)r : 0xffffffffu);
                    if (r == 0) best_s[n] = best;
                    if (rank == 0 && a.logits && r < V && (valid & (1u << n)))
                        a.logits[((size_t)(utt0 + n) * a.Tp + t) * V + r] = v;
                }
                __syncthreads();
                if (trp && tid == 0) trp[3] = clock64();
                // every thread keeps the counts; the token of utterance m is written by lane m of the last warp, which
                // has no part in the products that follow (one thread writing all eight held the whole cluster up)
                // (all decisions are read before any token is written: a shared-memory load may not pass a global store
                // that could alias it, and eight load -> compare -> store links in a row cost ~1 k cycles)
                emit = 0;
                int bests[M];
                {
                    const int4 b_lo = *reinterpret_cast<const int4*>(best_s), b_hi = *reinterpret_cast<const int4*>(best_s + 4);
                    bests[0] = b_lo.x; bests[1] = b_lo.y; bests[2] = b_lo.z; bests[3] = b_lo.w;
                    bests[4] = b_hi.x; bests[5] = b_hi.y; bests[6] = b_hi.z; bests[7] = b_hi.w;
                }
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const bool em = ((valid >> m) & 1u) && bests[m] != a.blank;
                    if (em && rank == 0 && tid == nthr - 32 + m) a.tokens[(size_t)(utt0 + m) * a.Tp + n_emit[m]] = bests[m];
                    n_emit[m] += em ? 1 : 0;
                    emit |= (em ? 1u : 0u) << m;
                }
            }
            if (emit) pred_eval(emit);
            else __syncthreads();
        }
        if (rank == 0 && tid == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m)
                if (valid & (1u << m)) a.n_tokens[utt0 + m] = n_emit[m];
        }
    }
    // After a wait that ran out, stores of a peer may still be on their way to this CTA (nothing waited for them):
    // give them time to land before anyone leaves.  The normal path has received everything that was sent to it.
    if (dead || status_aborted(a.status, a.gen))
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    cluster.sync();
}

using GreedyFn = void (*)(GreedyArgs);
// rows per warp are compile-time (register arrays); pick the instantiation covering the run-time sizes
// xb: the st.async exchange is possible (every CTA owns the same, even number of units)
static GreedyFn pick_greedy(int gate_rows, int joint_rows, int vocab, bool xb) {
    const int nrg = ceil_div(gate_rows, kGreedyWarps), nrj = ceil_div(joint_rows, kGreedyWarps),
              nrv = ceil_div(vocab, kGreedyWarps);
    if (nrg <= 5 && nrj <= 2 && nrv <= 2) return xb ? rnnt_greedy_kernel<5, 2, 2, true> : rnnt_greedy_kernel<5, 2, 2, false>;
    if (nrg <= kMaxRowsPerWarp && nrj <= 4 && nrv <= 4)
        return xb ? rnnt_greedy_kernel<kMaxRowsPerWarp, 4, 4, true> : rnnt_greedy_kernel<kMaxRowsPerWarp, 4, 4, false>;
    return nullptr;
}
static size_t greedy_mma_smem(const pimb200_rnnt_config& c, int C) {
    auto al = [](size_t b) { return (b + 15) & ~size_t(15); };
    const int PH = c.pred_hidden, JH = c.joint_hidden, M = kMmaUtts;
    const int RG = 4 * (PH / C);
    const int part_floats = 2 * M * RG > 4 * M * 32 ? 2 * M * RG : 4 * M * 32;
    return 3 * al((size_t)RG * PH * 2) + al((size_t)32 * JH * 2) + 2 * al((size_t)2 * M * (PH + 8) * 2) +
           al((size_t)M * JH * 2) + al((size_t)M * (JH + 8) * 2) + al((size_t)part_floats * 4) + al((size_t)M * 32 * 4) +
           al(32 * 4) + al((size_t)RG * 4) + al((size_t)M * 4) + al(6 * 8);
}
static bool greedy_mma_fits(const pimb200_rnnt_config& c, int C, int max_smem) {
    const int PH = c.pred_hidden, JH = c.joint_hidden;
    if (PH % C || JH % C || PH % 64 || JH % 64 || c.vocab > 32) return false;
    const int UP = PH / C, JP = JH / C;
    if ((4 * UP) % 16 || JP % 16) return false;
    if (3 * (4 * UP / 16) > kGreedyWarps || 4 * (JP / 16) > kGreedyWarps) return false;
    if (UP % 4 || JP % 8 || JP > 32 || UP > 32) return false;   // 8- / 16-byte chunks of the all-to-all copies; staging rows
    if (UP * kMmaUtts > kGreedyThreads || JP * kMmaUtts > kGreedyThreads) return false;
    return greedy_mma_smem(c, C) <= (size_t)max_smem;
}
constexpr int kGreedyMulti = 4;  // utterances per cluster of the lock-step variant
static GreedyFn pick_greedy_multi(int gate_rows, int joint_rows, int vocab) {
    const int nrg = ceil_div(gate_rows, kGreedyWarps), nrj = ceil_div(joint_rows, kGreedyWarps),
              nrv = ceil_div(vocab, kGreedyWarps);
    if (nrg <= 5 && nrj <= 2 && nrv <= 2) return rnnt_greedy_multi_kernel<5, 2, 2, kGreedyMulti>;
    return nullptr;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct pimb200_rnnt {
    pimb200_rnnt_config cfg;
    int device = 0;
    pimb200_lstm* pre = nullptr;
    pimb200_lstm* post = nullptr;
    __half *W1e = nullptr, *W1p = nullptr, *W2 = nullptr, *b1 = nullptr;
    uint4* W1pf = nullptr;          // W1p in the tensor-core kernel's fragment order, made once the cluster size is known
    float* b2 = nullptr;
    __half *Whh0 = nullptr, *Wih1 = nullptr, *Whh1 = nullptr;
    float *P0 = nullptr, *bias1 = nullptr;
    // workspace (grown on demand)
    __half *y_pre = nullptr, *y_post = nullptr;
    float* E = nullptr;
    size_t cap_frames = 0;  // frames*utts capacity of the three buffers above
    long long* trace = nullptr;  // diagnostics buffer (not owned)
    GreedyFn fn = nullptr;
    bool mma_ok = false;           // tensor-core variant (kMmaUtts utterances per cluster) available
    GreedyFn fn_mma = nullptr;     // its instantiation for this model's sizes
    size_t smem_bytes_mma = 0;
    GreedyFn fn_multi = nullptr;   // lock-step variant (kGreedyMulti utterances per cluster), when it fits
    int smem_mask_multi = 0;
    size_t smem_bytes_multi = 0;
    int greedy_multi = 1;   // 0 = always one utterance per cluster
    int enc_batch = 128;    // utterances the encoder advances in lock step
    int cluster = 0;        // CTAs per cluster
    int resident = 1;       // clusters of each greedy kernel that are co-resident on the device (occupancy query)
    int resident_mma = 1;
    int resident_multi = 1;
    int smem_mask = 0;
    size_t smem_bytes = 0;
    int* d_status = nullptr;        // status block of the greedy kernels' bounded waits: {sticky code, generation}
    int gen = 0;                    // generation of the last greedy launch
    int poll_limit = kGreedyPollLimit;
    std::mutex mu;
};

static size_t greedy_smem(const pimb200_rnnt_config& c, int C, int mask, int multi = 0) {
    auto al = [](size_t b) { return (b + 15) & ~size_t(15); };
    const int PH = c.pred_hidden, JH = c.joint_hidden, V = c.vocab;
    const int UP = (PH + C - 1) / C, JP = (JH + C - 1) / C;
    size_t s;
    if (multi > 0)
        s = al((size_t)multi * 2 * PH * 2) * 2 + al((size_t)multi * JH * 4) + al((size_t)multi * JH * 2) +
            al((size_t)multi * 4 * UP * 4) + al((size_t)multi * (V + 1) * 4) + al((size_t)V * 4) + al((size_t)4 * UP * 4);
    else
        s = al((size_t)2 * PH * 2) * 2 + al((size_t)JH * 4) + al((size_t)JH * 2) + al((size_t)4 * UP * 4) +
            al((size_t)(V + 1) * 4) + al((size_t)V * 4) + al((size_t)4 * UP * 4) + al((size_t)V * 4 * UP * 4) +
            al((size_t)UP * 2) + al(6 * 8);
    const size_t slice = al((size_t)4 * UP * PH * 2);
    if (mask & 1) s += slice;
    if (mask & 2) s += slice;
    if (mask & 4) s += slice;
    if (mask & 8) s += al((size_t)JP * PH * 2);
    if (mask & 16) s += al((size_t)V * JH * 2);
    return s;
}

extern "C" int pimb200_rnnt_destroy(pimb200_rnnt* h) {
    if (!h) return PIMB200_OK;
    cudaSetDevice(h->device);
    pimb200_lstm_destroy(h->pre);
    pimb200_lstm_destroy(h->post);
    void* ptrs[] = {h->W1e, h->W1p, h->W2, h->b1, h->b2, h->Whh0, h->Wih1, h->Whh1, h->P0, h->bias1,
                    h->y_pre, h->y_post, h->E, h->d_status, h->W1pf};
    for (void* p : ptrs) cudaFree(p);
    delete h;
    return PIMB200_OK;
}

extern "C" int pimb200_rnnt_create(const pimb200_rnnt_config* cfg, const pimb200_rnnt_weights* w,
                                   pimb200_rnnt** out) {
    if (!cfg || !w || !out) return PIMB200_ERR_BAD_ARG;
    const pimb200_rnnt_config c = *cfg;
    if (c.feat_dim <= 0 || c.enc_hidden <= 0 || c.pre_layers <= 0 || c.post_layers <= 0 || c.stack_factor <= 0 ||
        c.pred_hidden <= 0 || c.joint_hidden <= 0 || c.vocab <= 1 || c.blank < 0 || c.blank >= c.vocab)
        return PIMB200_ERR_BAD_ARG;
    if (!w->pre_params || !w->post_params || !w->pred_params || !w->embedding || !w->joint_w1 || !w->joint_b1 ||
        !w->joint_w2 || !w->joint_b2)
        return PIMB200_ERR_BAD_ARG;
    if (c.pred_layers != 2 || c.max_symbols != 1 || w->n_pred != 8) return PIMB200_ERR_UNSUPPORTED;
    if (c.pred_hidden % 8 || c.joint_hidden % 8 || c.joint_hidden > 1024 || c.vocab > 512) return PIMB200_ERR_UNSUPPORTED;
    pimb200_rnnt* h = new pimb200_rnnt();
    h->cfg = c;
    auto fail = [&](int code) { pimb200_rnnt_destroy(h); return code; };
    if (cudaGetDevice(&h->device) != cudaSuccess) return fail(PIMB200_ERR_LAUNCH);
    int rc;
    if ((rc = pimb200_lstm_create(w->pre_params, w->n_pre, c.pre_layers, 0, c.feat_dim, c.enc_hidden, 1, &h->pre)))
        return fail(rc);
    if ((rc = pimb200_lstm_create(w->post_params, w->n_post, c.post_layers, 0, c.stack_factor * c.enc_hidden,
                                  c.enc_hidden, 1, &h->post)))
        return fail(rc);
    const int EH = c.enc_hidden, PH = c.pred_hidden, JH = c.joint_hidden, V = c.vocab;
#define RNNT_ALLOC(ptr, bytes)                                                      \
    if (cudaMalloc(&(ptr), (bytes)) != cudaSuccess) return fail(PIMB200_ERR_NO_MEMORY)
    RNNT_ALLOC(h->W1e, (size_t)JH * EH * 2);
    RNNT_ALLOC(h->W1p, (size_t)JH * PH * 2);
    RNNT_ALLOC(h->W2, (size_t)V * JH * 2);
    RNNT_ALLOC(h->b1, (size_t)JH * 2);
    RNNT_ALLOC(h->b2, (size_t)V * 4);
    RNNT_ALLOC(h->Whh0, (size_t)4 * PH * PH * 2);
    RNNT_ALLOC(h->Wih1, (size_t)4 * PH * PH * 2);
    RNNT_ALLOC(h->Whh1, (size_t)4 * PH * PH * 2);
    RNNT_ALLOC(h->P0, (size_t)V * 4 * PH * 4);
    RNNT_ALLOC(h->bias1, (size_t)4 * PH * 4);
    RNNT_ALLOC(h->d_status, 8);
    if (cudaMemset(h->d_status, 0, 8) != cudaSuccess) return fail(PIMB200_ERR_LAUNCH);
    __half* wih0_packed = nullptr;
    float* bias0 = nullptr;
    RNNT_ALLOC(wih0_packed, (size_t)4 * PH * PH * 2);
    if (cudaMalloc(&bias0, (size_t)4 * PH * 4) != cudaSuccess) { cudaFree(wih0_packed); return fail(PIMB200_ERR_NO_MEMORY); }
#undef RNNT_ALLOC
    const size_t w1_pitch = (size_t)(EH + PH) * 2;
    cudaMemcpy2D(h->W1e, (size_t)EH * 2, w->joint_w1, w1_pitch, (size_t)EH * 2, JH, cudaMemcpyDeviceToDevice);
    cudaMemcpy2D(h->W1p, (size_t)PH * 2, static_cast<const __half*>(w->joint_w1) + EH, w1_pitch, (size_t)PH * 2, JH,
                 cudaMemcpyDeviceToDevice);
    cudaMemcpy(h->W2, w->joint_w2, (size_t)V * JH * 2, cudaMemcpyDeviceToDevice);
    cudaMemcpy(h->b1, w->joint_b1, (size_t)JH * 2, cudaMemcpyDeviceToDevice);
    rnnt_widen_kernel<<<ceil_div(V, 256), 256>>>(static_cast<const __half*>(w->joint_b2), h->b2, V);
    const void* const* pp = w->pred_params;  // (w_ih0, w_hh0, b_ih0, b_hh0, w_ih1, w_hh1, b_ih1, b_hh1)
    lstm_pack_matrix(static_cast<const __half*>(pp[0]), wih0_packed, PH, PH, nullptr);
    lstm_pack_matrix(static_cast<const __half*>(pp[1]), h->Whh0, PH, PH, nullptr);
    lstm_pack_matrix(static_cast<const __half*>(pp[4]), h->Wih1, PH, PH, nullptr);
    lstm_pack_matrix(static_cast<const __half*>(pp[5]), h->Whh1, PH, PH, nullptr);
    lstm_pack_bias(static_cast<const __half*>(pp[2]), static_cast<const __half*>(pp[3]), bias0, PH, nullptr);
    lstm_pack_bias(static_cast<const __half*>(pp[6]), static_cast<const __half*>(pp[7]), h->bias1, PH, nullptr);
    // P0[k] = W_ih0 . emb[k] + b_ih0 + b_hh0: one GEMM over the V embedding rows, then the bias on every row
    rc = launch_gemm_wx(wih0_packed, static_cast<const __half*>(w->embedding), nullptr, h->P0, 4 * PH, PH, V, PH,
                        4 * PH, PIMB200_ACT_NONE, 1, nullptr);
    rnnt_add_bias_rows_kernel<<<ceil_div(4 * PH * V, 256), 256>>>(h->P0, bias0, 4 * PH, V);
    cudaError_t e = cudaDeviceSynchronize();
    cudaFree(wih0_packed);
    cudaFree(bias0);
    if (rc != PIMB200_OK) return fail(rc);
    if (e != cudaSuccess) return fail(cuda_status(e));

    // cluster size and what fits in shared memory
    int max_smem = 0;
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, h->device);
    const int candidates[2] = {16, 8};
    for (int ci = 0; ci < 2 && h->cluster == 0; ++ci) {
        const int C = candidates[ci];
        GreedyFn fn = pick_greedy(4 * ceil_div(PH, C), ceil_div(JH, C), V, PH % C == 0 && (PH / C) % 2 == 0);
        if (!fn || C * ceil_div(PH, C) > kGreedyThreads) continue;   // one gate thread per (unit, destination CTA)
        cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
        int mask = 0;
        // stage in priority order while the budget lasts: W2 (read every frame) first, then the pred matrices
        const int order[5] = {16, 1, 2, 4, 8};
        for (int k = 0; k < 5; ++k)
            if (greedy_smem(c, C, mask | order[k]) <= (size_t)max_smem) mask |= order[k];
        const size_t smem = greedy_smem(c, C, mask);
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3(C);
        lc.blockDim = dim3(512);
        lc.dynamicSmemBytes = smem;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = C; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        lc.attrs = at;
        lc.numAttrs = 1;
        int n_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&n_clusters, fn, &lc) == cudaSuccess && n_clusters >= 1) {
            h->cluster = C;
            h->resident = n_clusters;
            h->fn = fn;
            h->smem_mask = mask;
            h->smem_bytes = smem;
            if (greedy_mma_fits(c, C, max_smem)) {
                // the benchmark model's sizes are compiled in; any other model takes them from the arguments
                GreedyFn fmma = (PH == 320 && JH == 512) ? rnnt_greedy_mma_kernel<320, 512> : rnnt_greedy_mma_kernel<0, 0>;
                cudaFuncSetAttribute(fmma, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                cudaFuncSetAttribute(fmma, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
                lc.dynamicSmemBytes = greedy_mma_smem(c, C);
                int ncl = 0;
                if (cudaOccupancyMaxActiveClusters(&ncl, fmma, &lc) == cudaSuccess && ncl >= 1) {
                    h->mma_ok = true;
                    h->fn_mma = fmma;
                    if (PH % 64 == 0 && cudaMalloc(&h->W1pf, (size_t)JH * PH * 2) == cudaSuccess) {
                        const int words = JH * PH / 2;
                        rnnt_pack_w1p_frags_kernel<<<ceil_div(words, 256), 256>>>(h->W1p, reinterpret_cast<uint32_t*>(h->W1pf),
                                                                                  JH, PH, C);
                        if (cudaDeviceSynchronize() != cudaSuccess) return fail(PIMB200_ERR_LAUNCH);
                    } else {
                        cudaGetLastError();
                        h->W1pf = nullptr;   // the kernel then reads the row-major matrix
                    }
                    h->resident_mma = ncl;
                    h->smem_bytes_mma = lc.dynamicSmemBytes;
                } else {
                    cudaGetLastError();
                }
            }
            // the lock-step variant needs kGreedyMulti sets of state buffers: use it only with every matrix resident
            GreedyFn fm = pick_greedy_multi(4 * ceil_div(PH, C), ceil_div(JH, C), V);
            const size_t smem_m = greedy_smem(c, C, 31, kGreedyMulti);
            if (fm && mask == 31 && smem_m <= (size_t)max_smem && ceil_div(PH, C) * kGreedyMulti <= kGreedyThreads) {
                cudaFuncSetAttribute(fm, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                cudaFuncSetAttribute(fm, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
                lc.dynamicSmemBytes = smem_m;
                int ncl = 0;
                if (cudaOccupancyMaxActiveClusters(&ncl, fm, &lc) == cudaSuccess && ncl >= 1) {
                    h->fn_multi = fm;
                    h->resident_multi = ncl;
                    h->smem_mask_multi = 31;
                    h->smem_bytes_multi = smem_m;
                } else {
                    cudaGetLastError();
                }
            }
        } else {
            cudaGetLastError();
        }
    }
    if (h->cluster == 0) return fail(PIMB200_ERR_UNSUPPORTED);
    *out = h;
    return PIMB200_OK;
}

extern "C" int pimb200_lstm_profile_enable(pimb200_lstm* h, int enable);
extern "C" int pimb200_lstm_profile_read(pimb200_lstm* h, double* total_ms, long* recurrences, double* bytes);

extern "C" int pimb200_rnnt_profile_enable(pimb200_rnnt* h, int enable) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    pimb200_lstm_profile_enable(h->pre, enable);
    return pimb200_lstm_profile_enable(h->post, enable);
}
extern "C" int pimb200_rnnt_profile_read(pimb200_rnnt* h, double* total_ms, long* recurrences, double* bytes) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    double ms[2] = {0, 0}, by[2] = {0, 0};
    long n[2] = {0, 0};
    int rc = pimb200_lstm_profile_read(h->pre, &ms[0], &n[0], &by[0]);
    if (rc != PIMB200_OK) return rc;
    rc = pimb200_lstm_profile_read(h->post, &ms[1], &n[1], &by[1]);
    if (rc != PIMB200_OK) return rc;
    if (total_ms) *total_ms = ms[0] + ms[1];
    if (recurrences) *recurrences = n[0] + n[1];
    if (bytes) *bytes = by[0] + by[1];
    return PIMB200_OK;
}

extern "C" int pimb200_rnnt_set_encoder_batch(pimb200_rnnt* h, int n) {
    if (!h || n < 1 || n > 128) return PIMB200_ERR_BAD_ARG;
    h->enc_batch = n;
    return PIMB200_OK;
}

// A/B switch: 0 = the greedy kernel always takes one utterance per cluster.
extern "C" int pimb200_rnnt_set_greedy_multi(pimb200_rnnt* h, int on) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    h->greedy_multi = on < 0 ? 0 : (on > 2 ? 2 : on);
    return PIMB200_OK;
}

extern "C" int pimb200_lstm_last_status(pimb200_lstm* h);
extern "C" int pimb200_lstm_set_poll_limit(pimb200_lstm* h, int limit);
extern "C" int pimb200_lstm_set_wavefront(pimb200_lstm* h, int on);
extern "C" int pimb200_gemm_last_status(void);

// First non-zero status word among the kernels a decode launches (both encoder stacks' recurrences, the tensor-core
// GEMMs of this device); reading clears them.  Synchronises the device.
extern "C" int pimb200_rnnt_last_status(pimb200_rnnt* h) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    const int s_pre = pimb200_lstm_last_status(h->pre);
    const int s_post = pimb200_lstm_last_status(h->post);
    const int s_gemm = pimb200_gemm_last_status();
    int s_greedy = PIMB200_OK;   // after the calls above the device is idle
    PIMB200_CUDA_TRY(cudaMemcpy(&s_greedy, h->d_status, 4, cudaMemcpyDeviceToHost));
    if (s_greedy != PIMB200_OK) PIMB200_CUDA_TRY(cudaMemset(h->d_status, 0, 4));
    return s_pre != PIMB200_OK ? s_pre : (s_post != PIMB200_OK ? s_post : (s_gemm != PIMB200_OK ? s_gemm : s_greedy));
}

// Test hook: the bounded waits of both encoder stacks (see pimb200_lstm_set_poll_limit).
extern "C" int pimb200_rnnt_set_poll_limit(pimb200_rnnt* h, int limit) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    const int rc = pimb200_lstm_set_poll_limit(h->pre, limit);
    if (rc != PIMB200_OK) return rc;
    h->poll_limit = limit < kGreedyPollLimit ? limit : kGreedyPollLimit;
    return pimb200_lstm_set_poll_limit(h->post, limit);
}

// A/B switch of both encoder stacks: layers in pairs as a wavefront for up to 8 utterances (see pimb200_lstm_set_wavefront).
extern "C" int pimb200_rnnt_set_wavefront(pimb200_rnnt* h, int on) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    const int rc = pimb200_lstm_set_wavefront(h->pre, on);
    return rc != PIMB200_OK ? rc : pimb200_lstm_set_wavefront(h->post, on);
}

// Diagnostics: device buffer of (T/stack)*8 int64 filled with per-frame clocks of utterance 0.
extern "C" int pimb200_rnnt_set_trace(pimb200_rnnt* h, long long* device_buffer) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    h->trace = device_buffer;
    return PIMB200_OK;
}

extern "C" int pimb200_rnnt_info(pimb200_rnnt* h, int* cluster_size, int* smem_mask, size_t* smem_bytes) {
    if (!h) return PIMB200_ERR_BAD_ARG;
    if (cluster_size) *cluster_size = h->cluster;
    if (smem_mask) *smem_mask = h->smem_mask;
    if (smem_bytes) *smem_bytes = h->smem_bytes;
    return PIMB200_OK;
}

template <typename T>
static int regrow(T** p, size_t elems) {
    if (*p) cudaFree(*p);
    *p = nullptr;
    PIMB200_CUDA_TRY(cudaMalloc(p, elems * sizeof(T)));
    return PIMB200_OK;
}

extern "C" int pimb200_rnnt_decode(pimb200_rnnt* h, const void* feats, int T, int n_utts, int32_t* tokens,
                                   int32_t* n_tokens, float* logits, void* stream) {
    if (!h || !feats || !tokens || !n_tokens || T <= 0 || n_utts <= 0) return PIMB200_ERR_BAD_ARG;
    const pimb200_rnnt_config& c = h->cfg;
    const int Tp = T / c.stack_factor;
    if (Tp <= 0) return PIMB200_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lk(h->mu);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int EH = c.enc_hidden, JH = c.joint_hidden;
    const size_t need = (size_t)n_utts * T;
    if (need > h->cap_frames) {
        PIMB200_CUDA_TRY(cudaDeviceSynchronize());
        int rc;
        if ((rc = regrow(&h->y_pre, need * EH))) return rc;
        if ((rc = regrow(&h->y_post, need * EH))) return rc;   // Tp*EH used
        if ((rc = regrow(&h->E, need * JH))) return rc;        // Tp*JH used
        h->cap_frames = need;
    }
    const __half* x = static_cast<const __half*>(feats);
    // The encoder runs up to `enc_batch` utterances in lock step (one column of the recurrence's tensor-core
    // tile each).  With batch-first tensors the time stacking between the two encoder stacks stays a pure
    // reinterpretation of memory: [g, T, EH] viewed as [g, T/stack, stack*EH] (T a multiple of stack).
    const int group = (T % c.stack_factor == 0) ? h->enc_batch : 1;
    for (int u = 0; u < n_utts; u += group) {
        const int g = (n_utts - u < group) ? (n_utts - u) : group;
        __half* y1 = h->y_pre + (size_t)u * T * EH;
        __half* y2 = h->y_post + (size_t)u * Tp * EH;
        int rc = pimb200_lstm_forward(h->pre, x + (size_t)u * T * c.feat_dim, T, g, nullptr, nullptr, y1, nullptr,
                                      nullptr, 1, stream);
        if (rc != PIMB200_OK) return rc;
        rc = pimb200_lstm_forward(h->post, y1, Tp, g, nullptr, nullptr, y2, nullptr, nullptr, 1, stream);
        if (rc != PIMB200_OK) return rc;
    }
    // encoder half of the joint for every frame of every utterance: one dense GEMM (y_post is contiguous over utts
    // only when T is a multiple of stack; handle the general case per utterance)
    if (T % c.stack_factor == 0 || n_utts == 1) {
        int rc = launch_gemm_wx(h->W1e, h->y_post, h->b1, h->E, JH, EH, n_utts * Tp, EH, JH, PIMB200_ACT_NONE, 1, st);
        if (rc != PIMB200_OK) return rc;
    } else {
        for (int u = 0; u < n_utts; ++u) {
            int rc = launch_gemm_wx(h->W1e, h->y_post + (size_t)u * Tp * EH, h->b1, h->E + (size_t)u * Tp * JH, JH,
                                    EH, Tp, EH, JH, PIMB200_ACT_NONE, 1, st);
            if (rc != PIMB200_OK) return rc;
        }
    }
    GreedyArgs a;
    a.E = h->E; a.tokens = tokens; a.n_tokens = n_tokens; a.logits = logits; a.n_utts = n_utts; a.Tp = Tp;
    a.P0 = h->P0; a.Whh0 = h->Whh0; a.Wih1 = h->Wih1; a.Whh1 = h->Whh1; a.bias1 = h->bias1;
    a.W1p = h->W1p; a.W1pf = h->W1pf; a.W2 = h->W2; a.b2 = h->b2;
    a.trace = h->trace;
    h->gen = h->gen == 0x7fffffff ? 1 : h->gen + 1;
    a.status = h->d_status; a.gen = h->gen; a.poll_limit = h->poll_limit;
    a.PH = c.pred_hidden; a.JH = JH; a.V = c.vocab; a.blank = c.blank; a.smem_mask = h->smem_mask;
    const int C = h->cluster;
    // more utterances than clusters: several utterances per cluster in lock step
    // greedy_multi: 0 = one utterance per cluster, 1 = best available, 2 = FMA lock-step variant (4 per cluster)
    const bool crowded = n_utts > h->resident;
    const bool use_mma = h->mma_ok && h->greedy_multi == 1 && crowded;
    const bool multi = !use_mma && h->fn_multi && h->greedy_multi >= 1 && crowded;
    const int groups = use_mma ? ceil_div(n_utts, kMmaUtts) : (multi ? ceil_div(n_utts, kGreedyMulti) : n_utts);
    // the grid holds as many clusters as are co-resident at this kernel's shared-memory footprint (the occupancy
    // query of create time), each working through groups cluster, cluster + n_clusters, ...
    const int max_clusters = use_mma ? h->resident_mma : (multi ? h->resident_multi : h->resident);
    const int n_clusters = groups < max_clusters ? groups : max_clusters;
    if (multi) a.smem_mask = h->smem_mask_multi;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(C * n_clusters);
    lc.blockDim = dim3(512);
    lc.dynamicSmemBytes = use_mma ? h->smem_bytes_mma : (multi ? h->smem_bytes_multi : h->smem_bytes);
    lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = C; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    lc.attrs = at;
    lc.numAttrs = 1;
    PIMB200_CUDA_TRY(cudaLaunchKernelEx(&lc, use_mma ? h->fn_mma : (multi ? h->fn_multi : h->fn), a));
    return PIMB200_OK;
}
