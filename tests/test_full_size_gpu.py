"""GPU checks at the sizes of the benchmark configuration (config 5: 64 x 256 tokens per micro-batch, E 1024, 16 heads,
FFN 4096, vocabulary 32000), where the CPU oracle would take minutes: each kernel is held to properties that do not
depend on the size -- rows of a softmax sum to one, masked positions are exactly zero, a LayerNorm's output is centred
and its input gradient is orthogonal to the constants, a product is linear in its operands, gradients of the loss sum
to zero over the vocabulary -- and to a plain fp32 PyTorch evaluation of the same formula where one fits in memory.

Tolerance: 1e-3 relative for everything that passes through the tf32 tensor cores, 1e-5 for the fp32 row kernels.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROWS, E, H, S, F, V = 64 * 256, 1024, 16, 256, 4096, 32000
TOL = 1e-3


@pytest.fixture(scope="module")
def capi(built):
    from opennn_b200 import capi as module
    module.lib()
    module.check(module.lib().onn_gemm_set_mode(0))
    torch.backends.cuda.matmul.allow_tf32 = False
    yield module
    assert module.lib().onn_gemm_device_status() == 0


def relative(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def test_dense_gemm_is_linear_and_matches_fp32(capi):
    """FFN-up shape on the two-CTA kernel: (A1 + A2) W = A1 W + A2 W, bias added once, and a strided sample of the
    output against an fp32 product."""
    g = torch.Generator(device="cuda").manual_seed(1)
    a1, a2 = (torch.randn(ROWS, E, device="cuda", generator=g) for _ in range(2))
    w = torch.randn(E, F, device="cuda", generator=g) / 32
    bias = torch.randn(F, device="cuda", generator=g)
    y1 = capi.dense_fwd(a1, w, bias, "Linear")
    y2 = capi.dense_fwd(a2, w, bias, "Linear")
    y12 = capi.dense_fwd(a1 + a2, w, bias, "Linear")
    assert relative(y12 + bias, y1 + y2) <= TOL
    rows = torch.arange(0, ROWS, 97, device="cuda")
    assert relative(y1[rows], a1[rows] @ w + bias) <= TOL


def test_relu_bits_and_masked_input_gradient(capi):
    """Dense(ReLU) -> Dense(Linear) at the FFN shapes: the bit mask written by the first layer's forward pass selects
    exactly the positive outputs, and the second layer's input gradient is zero exactly where they are not."""
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(ROWS, E, device="cuda", generator=g)
    w1 = torch.randn(E, F, device="cuda", generator=g) / 32
    w2 = torch.randn(F, E, device="cuda", generator=g) / 64
    b1, b2 = torch.zeros(F, device="cuda"), torch.zeros(E, device="cuda")
    y1, bits = capi.dense_fwd(x, w1, b1, "RectifiedLinear", want_relu_bits=True)
    y2 = capi.dense_fwd(y1, w2, b2, "Linear")
    unpacked = (bits.view(ROWS, F // 32, 1) >> torch.arange(32, device="cuda", dtype=torch.int32)) & 1
    assert torch.equal(unpacked.reshape(ROWS, F).bool(), y1 > 0)
    db1 = torch.zeros(F, device="cuda")
    delta = torch.randn(ROWS, E, device="cuda", generator=g)
    dx, dw2, db2 = capi.dense_bwd(y1, w2, y2, delta, "Linear", relu_bits=bits, dx_colsum=db1)
    assert torch.equal(dx != 0, (y1 > 0) & (dx != 0)) and float((dx[y1 <= 0]).abs().max()) == 0.0
    assert relative(db1, dx.sum(dim=0)) <= 1e-4
    assert relative(db2, delta.sum(dim=0)) <= 1e-4
    rows = torch.arange(0, ROWS, 131, device="cuda")
    assert relative(dx[rows], (delta[rows] @ w2.t()) * (y1[rows] > 0)) <= TOL


def test_layernorm_properties(capi):
    g = torch.Generator(device="cuda").manual_seed(3)
    x, r, dy = (torch.randn(ROWS, E, device="cuda", generator=g) for _ in range(3))
    gamma = torch.rand(E, device="cuda", generator=g) + 0.5
    beta = torch.randn(E, device="cuda", generator=g)
    y, mean, inv_std, total = capi.layernorm_fwd(x, gamma, beta, R=r, want_sum=True)
    assert torch.equal(total, x + r)
    normalised = (y - beta) / gamma
    assert float(normalised.mean(dim=1).abs().max()) <= 1e-5
    assert float((normalised.pow(2).mean(dim=1) - 1).abs().max()) <= 1e-4
    reference = torch.nn.functional.layer_norm(total, (E,), gamma, beta, eps=0.0)
    assert relative(y, reference) <= 1e-5
    sums = torch.zeros(E, device="cuda")
    dx, dgamma, dbeta = capi.layernorm_bwd(dy, total, mean, inv_std, gamma, dx_colsum=sums)
    # the input gradient of a LayerNorm is orthogonal to the constant vector and to the normalised input
    assert float(dx.sum(dim=1).abs().max()) <= 1e-3
    assert float((dx * normalised).sum(dim=1).abs().max()) <= 1e-2
    assert relative(dbeta, dy.sum(dim=0)) <= 1e-5
    assert relative(dgamma, (dy * normalised).sum(dim=0)) <= 1e-4
    assert relative(sums, dx.sum(dim=0)) <= 1e-4


@pytest.mark.parametrize("causal", [False, True])
def test_attention_layer_properties(capi, causal):
    """One attention layer of the benchmark's shape: rows of the weights sum to one, keys after the query (causal) and
    padded keys carry exactly zero weight, the context of a sample of strided rows matches fp32."""
    B = 64
    g = torch.Generator(device="cuda").manual_seed(4)
    p = {n: torch.randn(E, E, device="cuda", generator=g) * 0.03 for n in ("Wq", "Wk", "Wv", "Wo")}
    p.update({n: torch.randn(E, device="cuda", generator=g) * 0.01 for n in ("bq", "bk", "bv", "bo")})
    x = torch.randn(B, S, E, device="cuda", generator=g)
    x[:, S - 40:, :] = 0                                            # trailing padding: those keys are masked
    y, ws = capi.mha_fwd(x, x, p, H, causal)
    weights = capi.mha_attention_weights(ws, B, S, S, E, H)
    assert float((weights.sum(dim=-1) - 1).abs().max()) <= 1e-3
    assert float(weights[..., S - 40:].abs().max()) == 0.0
    if causal:
        above = torch.triu(torch.ones(S, S, device="cuda", dtype=torch.bool), diagonal=1)
        assert float(weights[:, :, above].abs().max()) == 0.0
    # sample (batch 5, head 3): fp32 evaluation of the same formula
    b, h, hd = 5, 3, E // H
    q = (x[b] @ p["Wq"] + p["bq"])[:, h * hd:(h + 1) * hd]
    k = (x[b] @ p["Wk"] + p["bk"])[:, h * hd:(h + 1) * hd]
    scores = q @ k.t() / np.sqrt(hd)
    scores[:, S - 40:] = -1e9
    if causal:
        scores = scores.masked_fill(above, float("-inf"))
    assert relative(weights[b, h], torch.softmax(scores, dim=-1)) <= TOL
    delta = torch.randn(B, S, E, device="cuda", generator=g)
    grads, dxq, _ = capi.mha_bwd(x, x, p, H, causal, ws, delta)
    assert relative(grads["dbo"], delta.reshape(-1, E).sum(dim=0)) <= 1e-4
    assert float(grads["dbk"].abs().max()) <= 1e-3 * float(grads["dbq"].abs().max())     # exactly zero in exact arithmetic
    assert torch.isfinite(dxq).all()


def test_cross_entropy_gradient_properties(capi):
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(ROWS, V, device="cuda", generator=g)
    targets = torch.randint(1, V, (ROWS,), device="cuda", generator=g).float()
    targets[::7] = 0                                                # padding targets: inactive rows
    active = targets > 0
    log_p = torch.log_softmax(logits[::64], dim=-1)                 # fp32 evaluation on a sample of rows
    error, accuracy, gradient, _ = capi.ce3d(logits, targets)       # in place: `logits` now holds the gradient
    assert float(gradient[~active].abs().max()) == 0.0
    assert float(gradient[active].sum(dim=-1).abs().max()) <= 1e-6
    count = int(active.sum())
    rows = torch.arange(0, ROWS, 64, device="cuda")
    sample_active = active[rows]
    expected = torch.exp(log_p)
    expected[torch.arange(len(rows), device="cuda"), targets[rows].long()] -= 1
    expected = expected / count
    assert relative(gradient[rows][sample_active], expected[sample_active]) <= 1e-5
    assert 0.0 <= accuracy <= 1.0 and abs(error - np.log(V)) < 1.0   # random logits: about log(V) + 1/2


def test_adam_without_gradient_leaves_parameters(capi):
    n = 50_000_000
    p = torch.randn(n, device="cuda")
    before = p.clone()
    m, v, g = (torch.zeros(n, device="cuda") for _ in range(3))
    sq = capi.grad_sqnorm(g)
    capi.adam(p, m, v, g, 2, sqnorm=sq, zero_grad=True)
    assert torch.equal(p, before) and float(m.abs().max()) == 0.0 and float(v.abs().max()) == 0.0
