"""Generates tests/golden/*.npz with libtorch CPU (fp32) — the library the reference's default
executors call for these ops (at::lstm, at::linear, at::addmm, at::matmul, at::cat).

Run from the repository root:  python tests/golden/make_golden.py
The fixtures pin oracle/oracle.c (CPU tests) and the CUDA kernels (GPU tests).  Inputs are
rounded to fp16-representable values first, so the fp16 device path consumes identical numbers.
torch version used for the committed files is stored in each fixture.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests.util import h16, lstm_params  # noqa: E402

# (name, T, B, I, H, L, bidirectional, has_biases, batch_first, nonzero_state)
LSTM_CASES = [
    ("lstm_t1_h8", 1, 1, 8, 8, 1, False, True, False, True),
    ("lstm_odd", 5, 3, 7, 5, 2, False, True, False, True),
    ("lstm_bi_bf", 6, 2, 16, 8, 2, True, True, True, True),
    ("lstm_nobias", 4, 1, 24, 16, 3, False, False, False, False),
    ("lstm_prenet_small", 12, 1, 240, 64, 2, False, True, False, False),
    ("lstm_pred_small", 2, 1, 320, 96, 2, False, True, False, True),
]
# (name, N, K, J, relu)
LINEAR_CASES = [
    ("linear_29x512", 29, 512, 1, False),
    ("linear_relu_64x1344", 64, 1344, 1, True),
    ("linear_tail_13x7", 13, 7, 1, False),
    ("linear_b8_40x96", 40, 96, 8, True),
]


def main():
    meta = dict(torch_version=torch.__version__)
    g = torch.Generator().manual_seed(1234)
    for (name, T, B, I, H, L, bi, hb, bf, nz) in LSTM_CASES:
        D = 2 if bi else 1
        ps = lstm_params(L, D, I, H, g, has_biases=hb)
        x = h16(torch.randn((B, T, I) if bf else (T, B, I), generator=g))
        h0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5) if nz else torch.zeros(L * D, B, H)
        c0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5) if nz else torch.zeros(L * D, B, H)
        y, hn, cn = torch.lstm(x, [h0, c0], ps, hb, L, 0.0, False, bi, bf)
        out = dict(x=x.numpy().astype(np.float16), h0=h0.numpy().astype(np.float16),
                   c0=c0.numpy().astype(np.float16), y=y.numpy(), hn=hn.numpy(), cn=cn.numpy(),
                   cfg=np.array([T, B, I, H, L, int(bi), int(hb), int(bf)]), **meta)
        for i, p in enumerate(ps):
            out[f"p{i}"] = p.numpy().astype(np.float16)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    # packed-sequence overload
    T, B, I, H, L = 7, 4, 12, 8, 2
    for bi in (False, True):
        D = 2 if bi else 1
        ps = lstm_params(L, D, I, H, g)
        lens = [7, 5, 5, 2]
        x = h16(torch.randn(T, B, I, generator=g))
        pk = torch.nn.utils.rnn.pack_padded_sequence(x, torch.tensor(lens))
        h0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5)
        c0 = h16(torch.randn(L * D, B, H, generator=g) * 0.5)
        y, hn, cn = torch.lstm(pk.data, pk.batch_sizes, [h0, c0], ps, True, L, 0.0, False, bi)
        out = dict(data=pk.data.numpy().astype(np.float16), batch_sizes=pk.batch_sizes.numpy(),
                   h0=h0.numpy().astype(np.float16), c0=c0.numpy().astype(np.float16), y=y.numpy(),
                   hn=hn.numpy(), cn=cn.numpy(), cfg=np.array([T, B, I, H, L, int(bi), 1, 0]), **meta)
        for i, p in enumerate(ps):
            out[f"p{i}"] = p.numpy().astype(np.float16)
        np.savez_compressed(os.path.join(HERE, f"lstm_packed_{'bi' if bi else 'uni'}.npz"), **out)
    for (name, N, K, J, relu) in LINEAR_CASES:
        k = 1.0 / (K ** 0.5)
        W = h16((torch.rand(N, K, generator=g) * 2 - 1) * k)
        b = h16((torch.rand(N, generator=g) * 2 - 1) * k)
        X = h16(torch.randn(J, K, generator=g))
        Y = torch.nn.functional.linear(X, W, b)
        if relu:
            Y = torch.relu(Y)
        # the same numbers through the addmm form the compiler rewrites linear into
        # (convert_linear_to_addmm.cpp:50-53 + swap_addmm_inputs.cpp:44-97): addmm(b, W, x^T)^T
        Y2 = torch.addmm(b.unsqueeze(1), W, X.t()).t()
        if relu:
            Y2 = torch.relu(Y2)
        assert torch.allclose(Y, Y2, atol=1e-5)
        # VM form on the transposed matrix: x[1,K] @ A[K,N]
        A = W.t().contiguous()
        Yvm = torch.matmul(X[0:1], A) + b
        if relu:
            Yvm = torch.relu(Yvm)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), W=W.numpy().astype(np.float16),
                            b=b.numpy().astype(np.float16), X=X.numpy().astype(np.float16), Y=Y.numpy(),
                            Yvm=Yvm.numpy(), relu=np.array(int(relu)), **meta)
    # add / cat
    A = h16(torch.randn(5, 44, generator=g))
    Bm = h16(torch.randn(5, 44, generator=g))
    Br = h16(torch.randn(44, generator=g))
    parts = [torch.randn(3, n, 4, generator=g).to(torch.float16) for n in (2, 5, 1)]
    np.savez_compressed(os.path.join(HERE, "glue.npz"), A=A.numpy().astype(np.float16),
                        B=Bm.numpy().astype(np.float16), Br=Br.numpy().astype(np.float16),
                        add_sym=(A.half() + Bm.half()).numpy(), add_bcast=(A.half() + Br.half()).numpy(),
                        cat0=parts[0].numpy(), cat1=parts[1].numpy(), cat2=parts[2].numpy(),
                        cat_out=torch.cat(parts, 1).numpy(), **meta)
    rowops(meta)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


def rowops(meta):
    """softmax / log_softmax / argmax / layer_norm / tanh / masked_fill over the last dimension (its own generator,
    so adding it left the older fixtures unchanged)."""
    g = torch.Generator().manual_seed(4321)
    out = dict(meta)
    for name, shape in (("logits", (3, 29)), ("scores", (8, 1, 13)), ("model", (5, 512)), ("vocab", (2, 1000))):
        x = h16(torch.randn(*shape, generator=g) * 3.0)
        out[f"{name}_x"] = x.numpy().astype(np.float16)
        out[f"{name}_softmax"] = torch.softmax(x, -1).numpy()
        out[f"{name}_log_softmax"] = torch.log_softmax(x, -1).numpy()
        out[f"{name}_argmax"] = torch.argmax(x, -1).numpy()
        out[f"{name}_tanh"] = torch.tanh(x).numpy()
    x = h16(torch.randn(5, 512, generator=g) * 2.0 + 0.5)
    gamma = h16(torch.rand(512, generator=g) + 0.5)
    beta = h16(torch.randn(512, generator=g) * 0.1)
    out["ln_x"], out["ln_gamma"], out["ln_beta"] = (t.numpy().astype(np.float16) for t in (x, gamma, beta))
    out["ln_y"] = torch.nn.functional.layer_norm(x, (512,), gamma, beta, 1e-5).numpy()
    out["ln_y_plain"] = torch.nn.functional.layer_norm(x, (512,), None, None, 1e-6).numpy()
    mask = torch.rand(4, 13, generator=g) < 0.3
    mx = h16(torch.randn(4, 13, generator=g))
    out["mf_x"], out["mf_mask"], out["mf_row_mask"] = mx.numpy().astype(np.float16), mask.numpy(), mask[0].numpy()
    out["mf_y"] = mx.masked_fill(mask, -65504.0).numpy()
    out["mf_y_row"] = mx.masked_fill(mask[0], 0.25).numpy()
    np.savez_compressed(os.path.join(HERE, "rowops.npz"), **out)


if __name__ == "__main__":
    main()
