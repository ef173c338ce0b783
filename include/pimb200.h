/*
 * pimb200.h — C ABI of libpimb200.so: the B200 (sm_100a) device back end for the
 * fp16 recurrent / decode hot path of PimAiCompiler's stream executor.
 *
 * Every entry point takes plain device pointers, sizes and an opaque stream
 * (a cudaStream_t passed as void*; NULL = the legacy default stream) and returns
 * an int status (PIMB200_OK == 0).  Nothing here owns or frees caller memory;
 * outputs may alias caller buffers at any 2-byte aligned offset (fast paths
 * engage when pointers are 16-byte aligned and the inner extent is a multiple
 * of 8 halves, other cases take a slower kernel — never a silent skip).
 *
 * All "half" pointers are IEEE fp16 device memory.  Arithmetic is fp16 storage,
 * fp32 accumulate, one rounding to fp16 at the op's output.
 *
 * Each declaration cites the interface of the reference it replaces
 * (paths relative to the PimAiCompiler tree).
 */
#ifndef PIMB200_H_
#define PIMB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
enum {
    PIMB200_OK = 0,
    PIMB200_ERR_BAD_ARG = 1,       /* null pointer, non-positive size, bad enum            */
    PIMB200_ERR_UNSUPPORTED = 2,   /* a shape this build has no kernel for                 */
    PIMB200_ERR_LAUNCH = 3,        /* CUDA reported an error at launch / sync              */
    PIMB200_ERR_TIMEOUT = 4,       /* a bounded device-side wait ran out (kernel returned) */
    PIMB200_ERR_NOT_INIT = 5,      /* pimb200_init() was not called for the current device */
    PIMB200_ERR_NO_MEMORY = 6      /* device allocation failed                             */
};

/* activation fused into the GEMV/GEMM epilogue.
 * Replaces PimActFunc{NONE, ACT_RELU} (runtime/source/executor/op_executor/aten_ops.cpp:614-622). */
enum { PIMB200_ACT_NONE = 0, PIMB200_ACT_RELU = 1 };

const char* pimb200_status_string(int status);

/* Library/device lifetime.  Replaces PimInitialize(RT_TYPE_HIP, PIM_FP16) / PimDeinitialize()
 * (runtime/source/nn_runtime.cpp:32, 85) and the rocBLAS warm-up (nn_runtime.cpp:62-73).
 * init allocates the per-device scratch used by the split-K GEMV; idempotent per device. */
int pimb200_init(int device);
int pimb200_shutdown(int device);

/* ---- batch-1 GEMV family ------------------------------------------------ */

/* MV:  y[N] = act(W[N,K] · x[K] + bias[N]);  W row-major, bias may be NULL.
 * Replaces the W_X_I PimExecuteGemm call of customAtenAddmm/customAtenMatmul
 * (aten_ops.cpp:662-694, 804-840) and rocblas_gemv_template_Axy / addmv_kernel_Axy
 * (runtime/include/executor/op_executor/custom_ops.h:141-214, 300-381). */
int pimb200_gemv_mv(const void* W, const void* x, const void* bias, void* y,
                    int N, int K, int act, void* stream);

/* VM:  y[N] = act(x[K] · A[K,N] + bias[N]);  A row-major K x N, bias may be NULL.
 * Replaces the I_X_W PimExecuteGemm call (aten_ops.cpp:626-661, 771-803) and
 * rocblas_gemv_template_xAy / addmv_kernel_xAy (custom_ops.h:66-139, 216-298).
 * Uses the per-device split-K scratch allocated by pimb200_init; calls on different streams are ordered by the
 * library, except launches captured into a CUDA graph: replays of such graphs must be ordered by the caller against
 * every other VM call on the device. */
int pimb200_gemv_vm(const void* x, const void* A, const void* bias, void* y,
                    int K, int N, int act, void* stream);

/* VM without any allocation: same result as pimb200_gemv_vm, for hosts that cannot let a plug-in allocate device
 * memory (a server that owns the whole device through its own arena, or a loop that cannot afford the device-wide
 * synchronisation of an allocation).  No counterpart in the reference.  The split-K scratch is a fixed array inside the
 * library image (about 1 MiB on every GPU that loads the library, held until exit); no pimb200_init is needed and no
 * call allocates or frees.  Limits: N <= PIMB200_VM_STATIC_MAX_N, K <= PIMB200_VM_STATIC_MAX_K, N a multiple of 8
 * and A 16-byte aligned; anything else returns PIMB200_ERR_UNSUPPORTED and launches nothing.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress): make that first call
 * outside any stream capture.  All calls on a device share the one array: calls that may overlap on the GPU (different
 * streams without ordering between them) race; order them, or use pimb200_gemv_vm. */
/* N bounds the scratch (partial sums and tickets are sized by the columns); K is only an argument sanity bound (row
 * indices are ints), no part of the scratch depends on it. */
#define PIMB200_VM_STATIC_MAX_N 32768
#define PIMB200_VM_STATIC_MAX_K 1048576
int pimb200_gemv_vm_static(const void* x, const void* A, const void* bias, void* y,
                           int K, int N, int act, void* stream);

/* VV:  y[0] = sum_k a[k]*b[k].  Replaces the VV branch of customAtenMatmul (aten_ops.cpp:841-882). */
int pimb200_dot_vv(const void* a, const void* b, void* y, int K, void* stream);

/* Single-row bmm:  y[n] = sum_k x[k]*A[k,n] (GNMT attention context, k = source length).
 * Replaces rocblas_bmm_template_xAy / bmm_kernel_xAy (custom_ops.h:435-466); accumulates in
 * fp32 (the reference kernel accumulates in fp16). */
int pimb200_bmm_row(const void* x, const void* A, void* y, int k, int n, void* stream);

/* Batched-stream GEMM:  Y[j, n] = act(sum_k X[j,k]*W[n,k] + bias[n]),  j < J.
 * X row-major [J, ldx>=K], W row-major [N,K], Y row-major [J, ldy>=N].
 * y_is_f32 != 0 stores fp32 (used for LSTM gate pre-activations), else fp16.
 * Replaces the MM-class fall-backs at::addmm / at::matmul / at::linear
 * (aten_ops.cpp:47-51, 304-307, 362, 695-711) and the MULTISTREAM fan-out
 * (runtime/source/executor/op_executor/stream_ops_executor.cpp:27-50). */
int pimb200_gemm_wx(const void* W, const void* X, const void* bias, void* Y,
                    int N, int K, int J, int ldx, int ldy, int act, int y_is_f32, void* stream);

/* n independent products of the form above in ONE launch when their shapes allow it (each with at most 32 activation
 * rows, or at most 256 against a matrix of at most 2048 rows; up to 8 per launch, more are issued in launches of 8); any
 * other mix is issued product by product on the same stream, so the call is always complete.  The fan-out of a
 * MULTISTREAM node (runtime/source/executor/op_executor/stream_ops_executor.cpp:27-50: N addmm / matmul layers, one host
 * thread and one stream each) as one grid: blockIdx.z is the branch. */
typedef struct pimb200_gemm_problem {
    const void* W;     /* [N, K] row-major */
    const void* X;     /* [J, ldx >= K] */
    const void* bias;  /* [N] or NULL */
    void* Y;           /* [J, ldy >= N] fp16, or fp32 when y_is_f32 */
    int N, K, J, ldx, ldy, act, y_is_f32;
} pimb200_gemm_problem;
int pimb200_gemm_wx_grouped(const pimb200_gemm_problem* problems, int n, void* stream);

/* Status of the tensor-core GEMM's bounded waits on the current device (0, or PIMB200_ERR_TIMEOUT if one gave up
 * since the last call); synchronises the device.  pimb200_gemm_force_simt(1) routes every pimb200_gemm_wx call
 * (and the LSTM input projections) to the SIMT kernel, for A/B profiling.  No counterpart in the reference. */
int pimb200_gemm_last_status(void);
int pimb200_gemm_force_simt(int on);

/* ---- glue ops ------------------------------------------------------------ */

/* C[m,n] = A[m,n] + B[m,n]   (broadcast_b == 0)   or   A[m,n] + B[n] (broadcast_b != 0).
 * C may alias A (the reference writes in place into A).  Any n (tail handled).
 * Replaces custom_add / add_kernel / add_kernel_unsym (custom_ops.h:383-433). */
int pimb200_add_f16(const void* A, const void* B, void* C, int m, int n, int broadcast_b, void* stream);

/* Strided 2-D copy of raw elements:  dst[r*dst_pitch + c] = src[r*src_pitch + c], r < rows, c < row_bytes
 * (pitches in bytes).  Building block for cat / copy_ into slices of a pre-allocated buffer.
 * Replaces atenCopy_ (aten_ops.cpp:126-129) on device tensors. */
int pimb200_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                    size_t row_bytes, size_t rows, void* stream);

/* Concatenate n_src row-major blocks along the inner dimension:
 * dst[o, off_i : off_i+inner_bytes[i]] = src[i][o, :], o < outer.  dst row pitch = sum(inner_bytes).
 * Replaces atenCat (aten_ops.cpp:97) for contiguous inputs. */
int pimb200_cat(void* dst, const void* const* src, const size_t* inner_bytes, int n_src,
                size_t outer, void* stream);

/* ---- row-wise glue of the decode path (fp16 storage, fp32 arithmetic), contiguous rows of `cols` elements ---- */

/* y[r, :] = softmax(x[r, :]) or log_softmax(x[r, :]) over the last dimension.
 * Replaces executeAtenSoftmax / executeAtenLogSoftmax -> at::softmax / at::log_softmax
 * (runtime/source/executor/op_executor/aten_ops_executor.cpp:3402-3436, 2092-2133; aten_ops.cpp:492, 323) for
 * dim = last. */
int pimb200_softmax_rows(const void* x, void* y, long rows, long cols, int log_softmax, void* stream);

/* idx[r] = index of the largest element of row r (the lowest index among equal maxima), int64.
 * Replaces executeAtenArgmax -> at::argmax (aten_ops_executor.cpp:520-547, aten_ops.cpp:71) for dim = last. */
int pimb200_argmax_rows(const void* x, long long* idx, long rows, long cols, void* stream);

/* y[r, :] = (x[r, :] - mean) / sqrt(var + eps) * gamma + beta, biased variance, over the last dimension;
 * gamma / beta [cols] fp16 or NULL.  Replaces executeAtenLayerNorm -> at::layer_norm
 * (aten_ops_executor.cpp:1898-1942, aten_ops.cpp:277-290) for a one-dimensional normalized_shape. */
int pimb200_layer_norm_rows(const void* x, const void* gamma, const void* beta, void* y, long rows, long cols, float eps,
                            void* stream);

/* y = tanh(x), n elements.  Replaces executeAtenTanh (aten_ops_executor.cpp:3555-3568). */
int pimb200_tanh_f16(const void* x, void* y, size_t n, void* stream);

/* y[i] = mask[i % mask_n] ? value : x[i]; mask holds one byte per element (bool), mask_n divides n (n = same shape,
 * cols = one mask row broadcast over the rows).  Replaces executeAtenMaskedFill with a scalar value
 * (aten_ops_executor.cpp:2432-2467, aten_ops.cpp:350-353). */
int pimb200_masked_fill_f16(const void* x, const unsigned char* mask, float value, void* y, size_t n, size_t mask_n,
                            void* stream);

/* The k largest (largest != 0) or smallest elements of every row of x [rows, cols] fp16, in order, and their int64
 * indices (equal values: lower index first): values [rows, k], idx [rows, k].  k <= 64.  The aten::topk of a decode
 * step over the last dimension (executeAtenTopk aten_ops_executor.cpp:3838, one at::topk call there). */
int pimb200_topk_rows(const void* x, void* values, long long* idx, long rows, long cols, int k, int largest, void* stream);

/* out[i, :] = table[idx[i], :] for n_idx int64 indices that live in DEVICE memory (rows of row_bytes bytes; an index
 * outside [0, n_table) gives a zero row).  The embedding lookup of a decode step without the host round trip of
 * executeAtenEmbedding, which reads the index with indices.item() (aten_ops_executor.cpp:1233-1300, the sync at
 * 1276-1287): the token chosen by pimb200_argmax_rows feeds the next step on the device. */
int pimb200_gather_rows(const void* table, const long long* idx, void* out, long n_idx, size_t row_bytes, long n_table,
                        void* stream);

/* table[idx[i], :] = src[i, :] for n_idx int64 row indices in DEVICE memory (indices outside [0, n_table) are skipped;
 * equal indices race).  This is aten::index_put_ along dimension 0 with whole rows as values and accumulate = false
 * (executeAtenIndexPut aten_ops_executor.cpp:1720), and the in-place KV-cache append of a decode step at a position kept on the device: where the
 * reference grows the cache with an at::cat per token (atenCat, aten_ops.cpp:97), the row goes into a pre-allocated
 * [S_max, d] buffer. */
int pimb200_scatter_rows(void* table, const long long* idx, const void* src, long n_idx, size_t row_bytes, long n_table,
                         void* stream);

/* Single-query multi-head attention of a decode step over a key / value cache:
 *     out[h, :] = softmax(scale * q[h, :] . K[0..L, h, :]^T) . V[0..L, h, :]   for each of `heads` heads,
 * q / out [heads * head_dim] fp16, K / V rows of kv_stride elements holding the heads side by side, attended length
 * L = (len_dev ? *len_dev : 0) + len_add clamped to [0, max_len]: len_dev is an int64 in DEVICE memory, so a step
 * captured in a CUDA graph attends to a cache that grows between replays.  max_len <= 8192.
 * Stands for the matmul -> (masked) softmax -> matmul group that the reference's Transformer graph executes as three
 * libtorch calls with per-head reshapes in between (executeAtenMatmul aten_ops_executor.cpp:2488-2505,
 * executeAtenSoftmax 3402-3436). */
int pimb200_attention_row(const void* q, const void* K, const void* V, const long long* len_dev, long len_add,
                          long max_len, void* out, int heads, int head_dim, long kv_stride, float scale, void* stream);

/* Batched form of pimb200_attention_row for n_seq sequences decoded in lock step: q / out are [n_seq, heads * head_dim],
 * sequence j attends to its own cache at K + j * seq_stride (V likewise) with its own length
 * L_j = (len_dev ? len_dev[j * len_inc] : 0) + len_add (len_inc 0: one shared device-side position, the self-attention
 * of a lock-step decode; len_inc 1: per-sequence source lengths, the cross-attention).  One launch, a CTA per
 * (head, sequence); rows of q / out are q_stride / out_stride elements apart.  The reference runs one sequence at a time (its matmul -> softmax -> matmul group, see above);
 * batching sentences is how one GPU serves many streams here. */
int pimb200_attention_rows(const void* q, const void* K, const void* V, const long long* len_dev, long len_inc,
                           long len_add, long max_len, void* out, int n_seq, int heads, int head_dim, long kv_stride,
                           long seq_stride, long q_stride, long out_stride, float scale, void* stream);

/* Multi-head self-attention over every position of n_seq padded sequences (a Transformer encoder layer):
 *     out[j, i, h, :] = softmax_s(scale * q[j, i, h, :] . k[j, s, h, :]) . v[j, s, h, :],   s < lengths[j] (int64, DEVICE;
 * NULL = max_len), for every query position i < lengths[j]; positions past the length give zero rows.  Row (j, i) of
 * q / k / v lies at j * seq_stride + i * row_stride elements (so the three may be column slices of one fused [.., 3d]
 * projection), of out at j * out_seq_stride + i * out_row_stride.  One launch, a CTA per (head, sequence), keys and
 * values of the head in shared memory (max_len * head_dim limited by 48 KB).  Stands for the per-head
 * matmul -> masked softmax -> matmul group of the reference's Transformer graph (executeAtenMatmul
 * aten_ops_executor.cpp:2488-2505, executeAtenMaskedFill, executeAtenSoftmax 3402-3436). */
int pimb200_attention_block(const void* q, const void* k, const void* v, const long long* lengths, void* out, int n_seq,
                            long max_len, int heads, int head_dim, long row_stride, long seq_stride, long out_row_stride,
                            long out_seq_stride, float scale, void* stream);

/* y = layer_norm(x + r) over the last dimension (gamma / beta optional): the residual add and the normalisation that
 * follow every Transformer sub-layer, two interpreter nodes in the reference (executeAtenAdd aten_ops_executor.cpp:110-166,
 * executeAtenLayerNorm).  cols * 4 bytes of shared memory per row. */
int pimb200_add_layer_norm_rows(const void* x, const void* r, const void* gamma, const void* beta, void* y, long rows,
                                long cols, float eps, void* stream);

/* Additive (normalised Bahdanau) attention of a GNMT decode step for n_seq sentences, one CTA per sentence:
 *     e[s] = sum_h v[h] * tanh(keys_proj[s, h] + q[h] + bias[h]),  s < lengths[j]  (int64 in DEVICE memory; NULL = max_len)
 *     ctx[j, :] = sum_s softmax(e)[s] * values[s, :]
 * q [n_seq, H]; row s of sentence j at j * seq_stride + s * row_stride elements of keys_proj / values (a time-major
 * encoder output [S, n_seq, H] has row_stride = n_seq * H, seq_stride = H); ctx rows ctx_stride elements apart, so the
 * context can be written straight into the second half of the decoder's [n_seq, 2H] concatenation buffer; `scores` is
 * caller-provided device scratch of n_seq * max_len floats (the raw scores e, left there).  Two launches.
 * Stands for the add -> tanh -> matmul -> softmax -> bmm chain of the reference's GNMT graph (executeAtenAdd
 * aten_ops_executor.cpp:110-166, executeAtenTanh, executeAtenMatmul 2488-2505, executeAtenSoftmax 3402-3436,
 * executeAtenBmm), five interpreter dispatches per token there. */
int pimb200_additive_attention(const void* q, const void* keys_proj, const void* values, const long long* lengths,
                               const void* v, const void* bias, void* ctx, float* scores, int n_seq, long max_len, int H,
                               long row_stride, long seq_stride, long ctx_stride, void* stream);

typedef struct pimb200_lstm pimb200_lstm;

/* One-time weight layout step.  params = the flat list at::lstm takes:
 * (w_ih[4H,I_l], w_hh[4H,H] [, b_ih[4H], b_hh[4H]]) per direction per layer, gate order i,f,g,o,
 * each a contiguous fp16 device buffer.  Packs gate-interleaved rows (row u*4+g) and the
 * summed bias in fp32 into memory owned by the handle.
 * Replaces ModelBuilder::buildLstmParameterVector / reArangeLstmWeights
 * (runtime/source/builder/model_builder.cpp:158-224, 226-319). */
int pimb200_lstm_create(const void* const* params, int n_params, int num_layers, int bidirectional,
                        int input_size, int hidden_size, int has_biases, pimb200_lstm** out);
int pimb200_lstm_destroy(pimb200_lstm* h);

/* variant selection for A/B profiling: 0 = automatic, 1 = streamed per-step kernels,
 * 2 = persistent weight-stationary kernels (one cooperative launch per layer and direction; W_hh slice in registers,
 * flag + bulk-copy exchange, 1..64 sequences, H a multiple of 16 up to 1024; larger H falls back to the variants with
 * W_hh in shared memory; fails with UNSUPPORTED when the shape does not fit), 3 = persistent with the tagged-word
 * exchange (W_hh in shared memory) for up to 8 sequences. */
enum { PIMB200_LSTM_AUTO = 0, PIMB200_LSTM_STREAMED = 1, PIMB200_LSTM_PERSISTENT = 2,
       PIMB200_LSTM_PERSISTENT_TAGGED = 3 };
int pimb200_lstm_set_variant(pimb200_lstm* h, int variant);

/* Forward pass, padded input:  x [T,B,I] (or [B,T,I] when batch_first), h0/c0 [L*D,B,H]
 * (NULL = zeros), y [T,B,D*H] (or [B,T,D*H]), hn/cn [L*D,B,H] (may be NULL).  Outputs must not overlap h0/c0.
 * Replaces atenLstm1 -> at::lstm (aten_ops.cpp:328-335) and executeMIOpenLSTM1's
 * miopenRNNForwardInference call (runtime/source/executor/op_executor/miopen_ops_executor.cpp:22-241).
 * y / hn / cn may point into slices of larger caller buffers (the reference's in-place
 * "custom cat" aliasing, miopen_ops_executor.cpp:193-228). */
int pimb200_lstm_forward(pimb200_lstm* h, const void* x, int T, int B, const void* h0, const void* c0,
                         void* y, void* hn, void* cn, int batch_first, void* stream);

/* One decode step (seq_len 1) of a one-layer, one-direction handle for B >= 8 sequences in lock step, with row strides:
 * x rows x_ld elements apart (a [B, x_ld] buffer whose first I columns are the input), the output written to rows y_ld
 * elements apart, optionally as y = h + residual (residual rows residual_ld apart; the fp16 add a separate aten::add of
 * the rounded h would make).  hn [B, H] receives h itself, cn [B, H] the cell state.  This is how the reference's GNMT
 * graph is wired after LstmLabeling / CatLabeling: a decoder cell writes its output straight into one half of the
 * pre-allocated buffer of the aten::cat that feeds the next cell (miopen_ops_executor.cpp:193-228) and the residual
 * aten::add works in place on it (aten_ops_executor.cpp:131-146); here both happen in the cell's gate kernel.  Shapes
 * outside the decode form (B < 8, more layers or directions, unaligned rows) return PIMB200_ERR_UNSUPPORTED: use
 * pimb200_lstm_forward. */
int pimb200_lstm_forward_step(pimb200_lstm* h, const void* x, long x_ld, int B, const void* h0, const void* c0, void* y,
                              long y_ld, void* hn, void* cn, const void* residual, long residual_ld, void* stream);

/* Forward pass, packed sequence:  data [sum(batch_sizes), I], batch_sizes = T host int64 values,
 * non-increasing; y [sum(batch_sizes), D*H]; h0/c0/hn/cn [L*D, batch_sizes[0], H].
 * Replaces atenLstm2 -> at::lstm(data, batch_sizes, ...) (aten_ops.cpp:337-344) and
 * executeMIOpenLSTM2 (miopen_ops_executor.cpp:243-421). */
int pimb200_lstm_forward_packed(pimb200_lstm* h, const void* data, const int64_t* batch_sizes, int T,
                                const void* h0, const void* c0, void* y, void* hn, void* cn, void* stream);

/* The last device-side status of a handle's asynchronous work: call after synchronising the
 * stream; returns PIMB200_ERR_TIMEOUT when a bounded wait inside the persistent kernel gave up (the outputs of that
 * call are then undefined); reading clears it.  A launch that gave up does not affect the launches after it. */
int pimb200_lstm_last_status(pimb200_lstm* h);

/* Timing hook: while enabled, every recurrence launch sequence (all T steps of one layer and direction)
 * is bracketed by CUDA events on the launching stream.  profile_read waits for those events and returns
 * their summed device time, how many recurrences ran and their algorithmic W_hh bytes
 * (T * 4H*H * 2 each: W_hh once per timestep; a launch of 65..128 sequences runs as two batch halves on separate
 * CTAs, each half a recurrence of its own with its own resident copy of W_hh, and counts twice), then clears the
 * record.  Stands where the reference wraps each op in
 * PROFILE_SCOPE + a device-wide sync (runtime/source/executor/stream_executor.cpp:204-258). */
int pimb200_lstm_profile_enable(pimb200_lstm* h, int enable);
int pimb200_lstm_profile_read(pimb200_lstm* h, double* total_ms, long* recurrences, double* bytes);

/* Opt-in A/B switch: 1 = run the recurrence of 17..64 lock-step sequences (H a multiple of 64) with tcgen05.mma and a
 * tensor-memory accumulator instead of mma.sync.  Same results; measured slower on B200 for this shape class (32 useful
 * rows per CTA), so the default is 0.  No counterpart in the reference. */
int pimb200_lstm_set_use_tc(pimb200_lstm* h, int on);

/* A/B switch between the batched persistent recurrences (lock-step sequences, H <= 1024): 2 (default) = the
 * pipelined kernel for 33..128 sequences (W_hh slice in registers; the sequences advance as independent groups, so
 * one group's hidden-state exchange runs under the other groups' arithmetic; 65..128 sequences as two batch halves)
 * and, for 1..32 sequences, the kernel with the exchange on the compute warps (shorter critical path when there is
 * nothing to overlap); 3 = the pipelined kernel for every batch size; 1 = the exchange-on-compute-warps kernel for
 * 1..64 sequences; 0 = the K-split kernel with W_hh in shared memory (up to 32 sequences; also what H > 1024 falls
 * back to).  Results agree within the LSTM tolerance; within one kernel they do not depend on the batch size.  No
 * counterpart in the reference. */
int pimb200_lstm_set_bulk_wide(pimb200_lstm* h, int on);

/* Tuning switch of the pipelined kernel: how many sequences form one independently advancing group (8, 16 or 32;
 * 0 = chosen by batch size, the default).  Same results.  No counterpart in the reference. */
int pimb200_lstm_set_pipe_group_size(pimb200_lstm* h, int seqs);

/* Packed input (pimb200_lstm_forward_packed) of up to 128 sequences and H % 16 == 0 runs as a padded lock-step batch on
 * the persistent recurrences (default, on = 1): the sequences are scattered into padded rows (the backward direction
 * reversed sequence by sequence), the gate terms behind a sequence's end freeze its cell state, outputs are gathered
 * back into packed rows.  on = 0 keeps the timestep-by-timestep streamed kernels (A/B and parity tests). */
int pimb200_lstm_set_packed_lockstep(pimb200_lstm* h, int on);

/* Stacked layers of a one-direction handle with up to 8 sequences (the batch-1 latency case) run in pairs as a wavefront
 * (default, on = 1): one cooperative launch advances layer l at timestep s and layer l + 1 at timestep s - 2 in the same
 * step, so a pair costs T + 2 dependent steps instead of 2T (H a multiple of 16 up to 1024, T >= 8).  Layer l + 1's
 * input product is then summed inside the recurrence instead of a hoisted GEMM: results agree with on = 0 within the
 * LSTM tolerance, not bit for bit. */
int pimb200_lstm_set_wavefront(pimb200_lstm* h, int on);

/* Shrinks (or restores) the iteration limit of the persistent kernel's bounded waits; used by the
 * fault-handling tests to see ERR_TIMEOUT quickly.  No counterpart in the reference, whose waits are
 * inside MIOpen. */
int pimb200_lstm_set_poll_limit(pimb200_lstm* h, int limit);

/* Tuning / diagnostics of the tagged-word persistent kernel (PIMB200_LSTM_PERSISTENT_TAGGED): how many replicas of the
 * exchange buffer every CTA publishes into (1..16) and how far apart consecutive exchange words lie, in 16-byte units
 * (1..8; 8 = one word per 128-byte line).  No counterpart in the reference. */
int pimb200_lstm_set_exchange_copies(pimb200_lstm* h, int copies);
int pimb200_lstm_set_exchange_stride(pimb200_lstm* h, int stride16);

/* Diagnostics: a device buffer of n_cta * T * 8 int64 that the persistent kernels fill with per-step clocks (NULL
 * switches it off).  Not owned by the handle.  No counterpart in the reference. */
int pimb200_lstm_set_trace(pimb200_lstm* h, long long* device_buffer);

#ifdef __cplusplus
}
#endif
#endif /* PIMB200_H_ */
