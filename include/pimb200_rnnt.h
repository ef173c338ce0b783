/*
 * pimb200_rnnt.h — C ABI of the device-resident RNN-T greedy decoder in libpimb200.so.
 *
 * The reference has no single function for this: it interprets the RNN-T TorchScript graph op by op
 * (StreamExecutor::inferenceModel, runtime/source/executor/stream_executor.cpp:136-202), the greedy
 * loop being a prim::Loop walked by the host (prim_ops_executor.cpp:744-922) around aten::embedding
 * (aten_ops_executor.cpp:1276-1287), two seq_len==1 aten::lstm calls, the split joint addmm pair
 * (compiler/include/frontend/optimizer/remove_cat_for_addmm.h:77-79) and an argmax read back per frame.
 * These entry points run the same arithmetic for one model family (RNN-T, greedy, at most one symbol per
 * frame) with the loop on the device.  Weights are passed exactly as the TorchScript constants hold them
 * (at::lstm flat parameter lists, nn.Linear weight/bias, nn.Embedding weight), fp16, device memory.
 */
#ifndef PIMB200_RNNT_H_
#define PIMB200_RNNT_H_

#include "pimb200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct pimb200_rnnt_config {
    int feat_dim;      /* 240  */
    int enc_hidden;    /* 1024 */
    int pre_layers;    /* 2    */
    int post_layers;   /* 3    */
    int stack_factor;  /* 2: consecutive frames concatenated between the two encoder stacks */
    int pred_hidden;   /* 320  */
    int pred_layers;   /* 2 (only value supported) */
    int joint_hidden;  /* 512  */
    int vocab;         /* 29, blank included */
    int blank;         /* 28; also the start-of-sequence input of the prediction network */
    int max_symbols;   /* 1 (only value supported) */
} pimb200_rnnt_config;

typedef struct pimb200_rnnt_weights {
    const void* const* pre_params;  int n_pre;   /* at::lstm list of LSTM(feat_dim -> enc_hidden, pre_layers)      */
    const void* const* post_params; int n_post;  /* at::lstm list of LSTM(stack*enc_hidden -> enc_hidden, post_layers) */
    const void* embedding;                       /* [vocab, pred_hidden]                                            */
    const void* const* pred_params; int n_pred;  /* at::lstm list of LSTM(pred_hidden -> pred_hidden, 2)           */
    const void* joint_w1; const void* joint_b1;  /* [joint_hidden, enc_hidden + pred_hidden], [joint_hidden]        */
    const void* joint_w2; const void* joint_b2;  /* [vocab, joint_hidden], [vocab]                                  */
} pimb200_rnnt_weights;

typedef struct pimb200_rnnt pimb200_rnnt;

/* Packs the weights (device-to-device) into memory owned by the handle. */
int pimb200_rnnt_create(const pimb200_rnnt_config* cfg, const pimb200_rnnt_weights* w, pimb200_rnnt** out);
int pimb200_rnnt_destroy(pimb200_rnnt* h);

/* Decodes n_utts utterances of T frames each: feats [n_utts, T, feat_dim] fp16.
 * tokens [n_utts, T/stack] int32 (emitted labels, in order), n_tokens [n_utts] int32,
 * logits (optional, may be NULL) [n_utts, T/stack, vocab] fp32 joint outputs of every frame.
 * Asynchronous on `stream`; all pointers are device memory. */
int pimb200_rnnt_decode(pimb200_rnnt* h, const void* feats, int T, int n_utts, int32_t* tokens,
                        int32_t* n_tokens, float* logits, void* stream);

/* How many utterances the encoder advances in lock step (1..128, default 128); each is one column of the
 * recurrence's tensor-core tiles.  1 reproduces strict batch-1 execution. */
int pimb200_rnnt_set_encoder_batch(pimb200_rnnt* h, int n);

/* Which greedy kernel a crowded call (more utterances than clusters) uses: 1 (default) = the best available
 * (tensor-core kernel, 8 utterances per cluster in lock step, when the shapes allow), 2 = the FMA lock-step kernel
 * (4 per cluster), 0 = always one utterance per cluster.  For A/B measurements. */
int pimb200_rnnt_set_greedy_multi(pimb200_rnnt* h, int mode);

/* Reports how the greedy kernel was configured: CTAs per cluster, which matrices are staged in shared
 * memory (bit 0..4 = W_hh0, W_ih1, W_hh1, joint W1 pred half, joint W2) and the dynamic shared memory per CTA. */
int pimb200_rnnt_info(pimb200_rnnt* h, int* cluster_size, int* smem_mask, size_t* smem_bytes);

/* pimb200_lstm_profile_enable / _read applied to both encoder stacks of the handle. */
int pimb200_rnnt_profile_enable(pimb200_rnnt* h, int enable);
int pimb200_rnnt_profile_read(pimb200_rnnt* h, double* total_ms, long* recurrences, double* bytes);

/* First non-zero status among the kernels a decode launched since the last call (PIMB200_ERR_TIMEOUT when a bounded
 * wait of a recurrence, of a tensor-core GEMM or of an exchange inside the greedy kernel gave up: the outputs of that
 * decode are then undefined); reading clears it.  Synchronises the device.  A timed-out launch does not affect later
 * launches. */
int pimb200_rnnt_last_status(pimb200_rnnt* h);

/* ---- diagnostics and test hooks (no counterpart in the reference) ---- */
/* Bounded waits of both encoder stacks and of the greedy kernel's exchange barriers, in polls (see
 * pimb200_lstm_set_poll_limit): fault tests shrink it to 1. */
int pimb200_rnnt_set_poll_limit(pimb200_rnnt* h, int limit);

/* pimb200_lstm_set_wavefront for both encoder stacks (default on). */
int pimb200_rnnt_set_wavefront(pimb200_rnnt* h, int on);
/* Device buffer of (T / stack_factor) * 8 int64 that the greedy kernel fills with per-frame clocks of utterance 0
 * (NULL switches it off).  Not owned by the handle. */
int pimb200_rnnt_set_trace(pimb200_rnnt* h, long long* device_buffer);

#ifdef __cplusplus
}
#endif
#endif /* PIMB200_RNNT_H_ */
