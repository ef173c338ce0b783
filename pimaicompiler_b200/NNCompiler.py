"""``NNCompiler.PipelineManager`` — the user-facing class of the reference's pybind module
(runtime/python/nn_runtime_py.cpp:18-25: ``PipelineManager(input_file, model_type="", gpu_num=1)`` with
``inferenceModel(input_tensors) -> List[Tensor]``), for the model family this library runs device-resident.

``model_type == "RNNT"``: ``input_file`` is a TorchScript file of an RNN-T module whose state dict has the entries
``pre_rnn.*``, ``post_rnn.*``, ``pred_embed.weight``, ``pred_rnn.*``, ``joint1.{weight,bias}``, ``joint2.{weight,bias}``
(``pimaicompiler_b200.synthetic.save_rnnt_torchscript`` writes one).  Inputs are ``[features [T,1,240] fp16,
feature_length int64]`` like the reference's RNN-T driver (examples/runtime/source/pipeline_manager.cpp:105-108);
the result list ends with the transcript (token ids), as the reference's RNN-T output tuple does.
``gpu_num > 1`` replicates the model: one worker thread and one handle per GPU, utterances dealt round-robin, results
returned in input order (the reference's thread-per-GPU scheme, runtime/python/pipeline_manager/pipeline_manager.cpp:27-53,
without its shared result vector).  Other model types need the TorchScript importer, which this library does not have.
"""
from __future__ import annotations

import threading
from typing import List, Sequence

import torch

from .synthetic import RnntConfig


def _lstm_list(sd, prefix: str, layers: int) -> List[torch.Tensor]:
    out = []
    for l in range(layers):
        out += [sd[f"{prefix}.weight_ih_l{l}"], sd[f"{prefix}.weight_hh_l{l}"], sd[f"{prefix}.bias_ih_l{l}"],
                sd[f"{prefix}.bias_hh_l{l}"]]
    return out


def _count_layers(sd, prefix: str) -> int:
    n = 0
    while f"{prefix}.weight_ih_l{n}" in sd:
        n += 1
    return n


class PipelineManager:
    def __init__(self, input_file: str, model_type: str = "", gpu_num: int = 1):
        if model_type != "RNNT":
            raise NotImplementedError(
                f"model_type {model_type!r}: only 'RNNT' runs device-resident here; other graphs need the TorchScript "
                "importer of the reference in front of the op executors")
        if not torch.cuda.is_available():
            raise RuntimeError("PipelineManager needs a CUDA device (there is no CPU fall-back)")
        from .rnnt import RnntDecoder
        self.model_type = model_type
        self.gpu_num = max(1, int(gpu_num))
        if self.gpu_num > torch.cuda.device_count():
            raise ValueError(f"gpu_num={gpu_num} but {torch.cuda.device_count()} devices are visible")
        module = torch.jit.load(input_file, map_location="cpu")
        sd = {k: v.detach() for k, v in module.state_dict().items()}
        pre_layers, post_layers = _count_layers(sd, "pre_rnn"), _count_layers(sd, "post_rnn")
        pred_layers = _count_layers(sd, "pred_rnn")
        enc_hidden = sd["pre_rnn.weight_hh_l0"].shape[1]
        feat = sd["pre_rnn.weight_ih_l0"].shape[1]
        stack = sd["post_rnn.weight_ih_l0"].shape[1] // enc_hidden
        vocab, pred_hidden = sd["pred_embed.weight"].shape
        self.cfg = RnntConfig(feat_dim=feat, enc_hidden=enc_hidden, pre_layers=pre_layers, post_layers=post_layers,
                              stack_factor=stack, pred_hidden=pred_hidden, pred_layers=pred_layers,
                              joint_hidden=sd["joint1.weight"].shape[0], vocab=vocab, blank=vocab - 1, max_symbols=1)
        self.decoders = []
        for g in range(self.gpu_num):
            dev = torch.device("cuda", g)
            d = lambda t: t.to(torch.float16).to(dev).contiguous()
            with torch.cuda.device(dev):
                self.decoders.append(RnntDecoder(
                    self.cfg, [d(t) for t in _lstm_list(sd, "pre_rnn", pre_layers)],
                    [d(t) for t in _lstm_list(sd, "post_rnn", post_layers)], d(sd["pred_embed.weight"]),
                    [d(t) for t in _lstm_list(sd, "pred_rnn", pred_layers)], d(sd["joint1.weight"]),
                    d(sd["joint1.bias"]), d(sd["joint2.weight"]), d(sd["joint2.bias"])))

    def _decode_on(self, g: int, feats: torch.Tensor):
        dev = torch.device("cuda", g)
        with torch.cuda.device(dev):
            f = feats.to(dev, torch.float16).contiguous()
            toks, logits = self.decoders[g].decode(f, want_logits=True)
            torch.cuda.synchronize(dev)
        return toks, logits

    def inferenceModel(self, input_tensors: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        """``[features, feature_length]`` -> ``[logits [Tp, vocab] fp32, n_tokens, transcript int64]`` on cuda:0.

        ``features`` is time-major ``[T, B, feat]``; with B > 1 the utterances are sharded over the GPUs and the
        outputs are lists flattened utterance by utterance."""
        feats = input_tensors[0]
        if feats.dim() != 3:
            raise ValueError("features must be [T, B, feat_dim]")
        T = int(input_tensors[1].reshape(-1)[0]) if len(input_tensors) > 1 else feats.shape[0]
        feats = feats[:T].transpose(0, 1).contiguous()  # [B, T, F]
        B = feats.shape[0]
        shards = [list(range(g, B, self.gpu_num)) for g in range(self.gpu_num)]
        results = [None] * B
        errors = []

        def work(g):
            try:
                if not shards[g]:
                    return
                toks, logits = self._decode_on(g, feats[shards[g]])
                for k, u in enumerate(shards[g]):
                    results[u] = (toks[k], logits[k])
            except Exception as e:  # surfaced to the caller after the join
                errors.append((g, e))

        if self.gpu_num == 1:
            work(0)
        else:
            threads = [threading.Thread(target=work, args=(g,)) for g in range(self.gpu_num)]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
        if errors:
            raise RuntimeError(f"replica on cuda:{errors[0][0]} failed: {errors[0][1]}") from errors[0][1]
        out: List[torch.Tensor] = []
        for toks, logits in results:
            out += [logits.to("cuda:0"), torch.tensor([len(toks)], device="cuda:0"),
                    torch.tensor(toks, dtype=torch.int64, device="cuda:0")]
        return out
