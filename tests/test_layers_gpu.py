"""GPU parity: every layer entry point of the C ABI against the golden fixtures produced by
the unmodified reference CPU library (same seeded inputs).  Shapes are the reference's own
layer-test shapes plus config 1; ragged, padded and out-of-range cases included.

Tolerance: 1e-3 (max-abs and L2, relative) for anything that passes through the tf32
tensor cores; embedding values are compared bit for bit.
"""

import glob
import os

import numpy as np
import pytest
import torch

from tests.util import GOLDEN, TOL, assert_close, errors, golden
from tests.golden.make_golden import mha_unpack

pytestmark = pytest.mark.gpu


def names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def host(t):
    return t.detach().cpu().numpy()


@pytest.fixture(scope="module")
def capi(built):
    from opennn_b200 import capi as module
    module.lib()
    yield module
    module.check(module.lib().onn_gemm_set_mode(0))


@pytest.fixture(params=["auto", "simt"])
def gemm_mode(request, capi):
    """auto = tcgen05 wherever the TMA alignment rules allow it; simt = CUDA-core cross-check."""
    capi.check(capi.lib().onn_gemm_set_mode(1 if request.param == "simt" else 0))
    yield request.param
    assert capi.lib().onn_gemm_device_status() == 0, "a tcgen05 GEMM gave up on a bounded wait"
    capi.check(capi.lib().onn_gemm_set_mode(0))


# ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", names("embedding_"))
def test_embedding(capi, name):
    g = golden(name)
    B, S, V, E, scale, add_pe = (int(v) for v in g["spec"])
    ids, W, pe = dev(g["ids"]), dev(g["weights"]), dev(g["pe"])
    y, flags = capi.embedding_fwd(ids, W, pe, bool(scale), bool(add_pe), want_flags=True)
    assert np.array_equal(host(y).view(np.uint32), g["y"].view(np.uint32)), "embedding forward must be bit-exact"
    expected_flags = np.all(np.abs(g["y"]) <= 1e-7, axis=-1).reshape(-1)
    assert np.array_equal(host(flags).astype(bool), expected_flags)
    dW = capi.embedding_bwd(ids, dev(g["delta"]), V, bool(scale))
    assert_close(host(dW), g["dW"], 1e-5, "dW")
    assert not host(dW)[0].any(), "padding row gradient must be exactly zero"
    # fan-in sum of two consumer gradients
    half = dev(g["delta"] * 0.5)
    dW2 = capi.embedding_bwd(ids, half, V, bool(scale), dY2=half)
    assert_close(host(dW2), g["dW"], 1e-5, "dW with two consumers")


@pytest.mark.parametrize("name", names("layernorm_"))
def test_layernorm(capi, name):
    g = golden(name)
    x, gamma, beta, delta = dev(g["x"]), dev(g["gammas"]), dev(g["betas"]), dev(g["delta"])
    y, mean, inv_std, _ = capi.layernorm_fwd(x, gamma, beta)
    assert_close(host(y), g["y"], 1e-5, "y")
    dx, dgamma, dbeta = capi.layernorm_bwd(delta, x, mean, inv_std, gamma)
    assert_close(host(dx), g["dx"], 5e-5, "dx")
    assert_close(host(dgamma), g["dgamma"], 5e-5, "dgamma")
    assert_close(host(dbeta), g["dbeta"], 5e-5, "dbeta")
    # column sums of dx, ADDED to a caller's vector: the bias gradient of the layer whose output was normalised
    E = g["x"].shape[-1]
    sums = torch.ones(E, device="cuda")
    dx_again, _, _ = capi.layernorm_bwd(delta, x, mean, inv_std, gamma, dx_colsum=sums)
    assert np.array_equal(host(dx_again), host(dx))
    expected_sums = 1.0 + g["dx"].reshape(-1, E).astype(np.float64).sum(axis=0)
    assert_close(host(sums), expected_sums, 5e-5, "column sums of dx", floor=float(np.abs(g["dx"]).reshape(-1, E).sum(axis=0).max()) * 1e-1)
    # fused residual add: A + R = x, and the sum comes back as the Addition layer's output
    a = dev(g["x"] * 0.25)
    r = dev(g["x"] - g["x"] * 0.25)
    y2, mean2, inv_std2, total = capi.layernorm_fwd(a, gamma, beta, R=r, want_sum=True)
    assert_close(host(total), host(a) + host(r), 1e-7, "sum")
    assert_close(host(y2), g["y"], 2e-5, "y (fused add)")
    # fan-in sum of three consumer gradients
    third = dev(g["delta"] / 4)
    dx3, dgamma3, _ = capi.layernorm_bwd(third, x, mean, inv_std, gamma, dY2=third, dY3=dev(g["delta"] / 2))
    assert_close(host(dx3), g["dx"], 5e-5, "dx (three consumers)")
    assert_close(host(dgamma3), g["dgamma"], 5e-5, "dgamma (three consumers)")


@pytest.mark.parametrize("name", names("pooling_"))
def test_pooling3d(capi, name):
    """Sequence pooling against the reference's outputs: padding rows, a sample of nothing but padding, a tie for the
    maximum.  Element-wise work in the reference's order: bit-exact."""
    g = golden(name)
    method = str(g["method"])
    x = dev(g["x"])
    y, saved = capi.pooling3d_fwd(x, method)
    assert np.array_equal(host(y), g["y"]), "y"
    dx = capi.pooling3d_bwd(dev(g["delta"]), saved, g["x"].shape[1], method)
    assert np.array_equal(host(dx), g["dx"]), "dx"


@pytest.mark.parametrize("name", names("dense_"))
def test_dense(capi, gemm_mode, name):
    g = golden(name)
    activation = str(g["activation"])
    x, W, b, delta = dev(g["x"]), dev(g["weights"]), dev(g["biases"]), dev(g["delta"])
    y = capi.dense_fwd(x, W, b, activation)
    assert_close(host(y), g["y"], TOL, "y")
    dx, dW, db = capi.dense_bwd(x, W, y, delta, activation)
    expected = {"dx": g["dx"], "dW": g["dW"], "db": g["db"]}
    if activation == "RectifiedLinear" and gemm_mode == "auto":
        # A pre-activation within tf32 rounding distance of zero may land on the other side of the ReLU
        # kink, which flips that element's derivative whatever the precision.  Masks may differ only
        # there; everything else is compared with the device's mask applied to the reference delta.
        from oracle import opennn_oracle as O
        reference_mask = g["y"].reshape(host(y).shape) > 0
        device_mask = host(y) > 0
        disagree = reference_mask != device_mask
        assert disagree.mean() <= 5e-3
        assert np.abs(g["y"].reshape(host(y).shape)[disagree]).max(initial=0.0) <= 2e-3 * np.abs(g["y"]).max()
        dx_e, dW_e, db_e = O.dense_backward(g["x"], g["weights"], g["delta"], device_mask.astype(np.float32), activation)
        expected = {"dx": dx_e, "dW": dW_e, "db": db_e}
    assert_close(host(dx), expected["dx"], TOL, "dx")
    assert_close(host(dW), expected["dW"], TOL, "dW")
    assert_close(host(db), expected["db"], TOL, "db")


@pytest.mark.parametrize("rows,features,hidden", [(96, 40, 72), (1024, 256, 512)])
def test_dense_pair_relu_bits(capi, gemm_mode, rows, features, hidden):
    """Feed-forward pair Dense(ReLU) -> Dense(Linear): the first layer's forward pass writes (y > 0) as bits, the
    second layer's backward pass applies them to its input gradient and takes the first layer's bias gradient
    from the column sums.  The result must be the one the float mask gives, and match the layer-by-layer oracle."""
    from oracle import opennn_oracle as O
    rng = np.random.default_rng(rows + hidden)
    x = rng.standard_normal((rows, features)).astype(np.float32)
    W1 = (rng.standard_normal((features, hidden)) / np.sqrt(features)).astype(np.float32)
    b1 = (0.1 * rng.standard_normal(hidden)).astype(np.float32)
    W2 = (rng.standard_normal((hidden, features)) / np.sqrt(hidden)).astype(np.float32)
    b2 = (0.1 * rng.standard_normal(features)).astype(np.float32)
    delta = rng.standard_normal((rows, features)).astype(np.float32)

    y1, bits = capi.dense_fwd(dev(x), dev(W1), dev(b1), "RectifiedLinear", want_relu_bits=True)
    y2 = capi.dense_fwd(y1, dev(W2), dev(b2), "Linear")
    db1_bits = torch.zeros(hidden, device="cuda")
    dx_bits, dW2, db2 = capi.dense_bwd(y1, dev(W2), y2, dev(delta), "Linear", relu_bits=bits, dx_colsum=db1_bits)
    db1_mask = torch.zeros(hidden, device="cuda")
    dx_mask, _, _ = capi.dense_bwd(y1, dev(W2), y2, dev(delta), "Linear", relu_mask=y1, dx_colsum=db1_mask)
    assert np.array_equal(host(dx_bits), host(dx_mask)), "bit mask and float mask must select the same elements"
    assert_close(host(db1_bits), host(db1_mask), 1e-5, "db1 from column sums")

    device_mask = (host(y1) > 0).astype(np.float32)
    dy1, dW2_e, db2_e = O.dense_backward(host(y1), W2, delta, np.ones_like(delta), "Linear")
    assert_close(host(dx_bits), dy1 * device_mask, TOL, "delta of the ReLU layer")
    assert_close(host(dW2), dW2_e, TOL, "dW2")
    assert_close(host(db2), db2_e, TOL, "db2")
    assert_close(host(db1_bits), (dy1 * device_mask).sum(axis=0), TOL, "db1", floor=1e-3 * np.abs(dy1).sum(axis=0).max())


@pytest.mark.parametrize("name", names("mha_"))
def test_mha(capi, gemm_mode, name):
    g = golden(name)
    B, Sq, Sk, E, H, causal, cross = (int(v) for v in g["spec"])
    p = {k: dev(v) for k, v in mha_unpack(g["params"], E).items()}
    xq = dev(g["xq"])
    xs = dev(g["xs"]) if cross else xq
    y, ws = capi.mha_fwd(xq, xs, p, H, bool(causal))
    assert_close(host(y), g["y"], TOL, "y")
    weights = capi.mha_attention_weights(ws, B, Sq, Sk, E, H)
    assert_close(host(weights), g["attention_weights"], TOL, "attention weights")
    grads, dxq, dxs = capi.mha_bwd(xq, xs, p, H, bool(causal), ws, dev(g["delta"]))
    assert_close(host(dxq), g["dxq"], TOL, "dxq")
    if cross:
        assert_close(host(dxs), g["dxs"], TOL, "dxs")
    ref = mha_unpack(g["grads"], E)
    floor = float(np.abs(g["grads"]).max())
    # tf32 unit round-off is 4.9e-4 per operand, so one product carries up to 9.8e-4: with reductions of
    # a handful of terms (these shapes have head size 4 and 3 to 16 keys) a single element can touch
    # 1e-3, which is why the per-view bound is on the L2 error and the whole arena is judged on both
    device_arena = np.concatenate([host(grads["d" + key]).ravel() for key in ref])
    reference_arena = np.concatenate([value.ravel() for value in ref.values()])
    arena_max, arena_l2 = errors(device_arena, reference_arena)
    if arena_max > TOL:
        print(f"\n[{name}/{gemm_mode}] parameter gradients: largest element error {arena_max:.2e} (l2 {arena_l2:.2e})")
    assert_close(device_arena, reference_arena, TOL if gemm_mode == "simt" else 2 * TOL, "parameter gradients")
    for key, value in ref.items():
        _, l2 = errors(host(grads["d" + key]), value, floor=floor)
        assert l2 <= TOL, f"d{key}: l2-rel {l2:.3e}"


@pytest.mark.parametrize("name", names("ce3d_"))
def test_ce3d(capi, name):
    g = golden(name)
    targets = dev(g["targets"])
    # from logits (fused softmax), the training path
    error, accuracy, grad, p = capi.ce3d(dev(g["logits"]), targets, want_probabilities=True)
    assert abs(error - g["loss"][0]) <= 1e-5 * max(1.0, abs(g["loss"][0]))
    assert abs(accuracy - g["loss"][1]) <= 1e-6
    assert_close(host(grad), g["dlogits"], 1e-5, "dlogits")
    assert_close(host(p), g["p"], 1e-5, "probabilities")
    # from probabilities, as a plain Softmax Dense layer leaves them
    error2, accuracy2, grad2, _ = capi.ce3d(dev(g["p"]), targets, inputs_are_probabilities=True)
    assert abs(error2 - g["loss"][0]) <= 1e-6 * max(1.0, abs(g["loss"][0]))
    assert accuracy2 == accuracy
    assert_close(host(grad2), g["dlogits"], 1e-6, "dlogits from probabilities")


def test_ce3d_all_masked(capi):
    logits = torch.randn(2, 3, 16, device="cuda")
    targets = torch.zeros(2, 3, device="cuda")
    error, accuracy, grad, _ = capi.ce3d(logits, targets)
    assert error == 0.0 and accuracy == 0.0 and not host(grad).any()


@pytest.mark.parametrize("rows,V", [(5, 4096), (301, 4100), (200, 8000), (333, 32000), (40, 35712), (9, 35716), (7, 51584)])
def test_ce3d_long_rows(capi, rows, V):
    """Rows of 4096 to 35712 logits are held in registers by the persistent kernel, fed through a ring of 3968-float
    chunks in shared memory (V = 4100 ends in a 132-float chunk, 8000 takes the 3-chunk instantiation, 35712 is nine full
    chunks; 35716 and 51584 are past it and fall back to the two-sweep kernel).
    Against the restated reference arithmetic and against the two-sweep kernel on the same inputs: padding targets,
    targets past the vocabulary, a row with two equal maxima (the first one counts), logits and probabilities as input."""
    from oracle import opennn_oracle as O
    ONN_CE_TWO_SWEEPS = 32
    rng = np.random.default_rng(rows * 131 + V)
    logits = (3.0 * rng.standard_normal((1, rows, V))).astype(np.float32)
    targets = rng.integers(1, V, size=(1, rows)).astype(np.float32)
    targets[0, ::5] = 0                                   # padding
    targets[0, 3] = V + 7                                 # past the vocabulary: inactive
    if rows > 8:
        top = float(logits[0, 6].max()) + 1.0             # two equal maxima far apart: arg-max is the first
        logits[0, 6, V - 3] = top
        logits[0, 6, 17] = top
        targets[0, 6] = 17
        targets[0, 7] = float(V - 1)                      # the very last logit of a row
    shifted = logits - logits.max(axis=-1, keepdims=True)
    p = np.exp(shifted, dtype=np.float32)
    p = (p / p.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)
    expected_error, expected_accuracy, count = O.ce3d_error(p, targets)
    expected_gradient = O.ce3d_output_gradients(p, targets)

    error, accuracy, gradient, _ = capi.ce3d(dev(logits), dev(targets))
    error2, accuracy2, gradient2, _ = capi.ce3d(dev(logits), dev(targets), flags=ONN_CE_TWO_SWEEPS)
    assert abs(error - expected_error) <= 1e-5 * abs(expected_error)
    assert abs(accuracy - expected_accuracy) <= 1e-6 and accuracy == accuracy2
    assert abs(error - error2) <= 1e-6 * abs(error2)
    assert_close(host(gradient), expected_gradient, 1e-5, "dlogits")
    assert_close(host(gradient), host(gradient2), 1e-5, "dlogits, staged against two sweeps")
    inactive = ~((targets[0] > 0) & (targets[0] < V))
    assert not host(gradient)[0, inactive].any()

    error3, accuracy3, gradient3, _ = capi.ce3d(dev(p), dev(targets), inputs_are_probabilities=True)
    assert abs(error3 - expected_error) <= 1e-6 * abs(expected_error) and accuracy3 == accuracy
    assert_close(host(gradient3), expected_gradient, 1e-6, "dlogits from probabilities")
    assert capi.lib().onn_gemm_device_status() == 0


@pytest.mark.parametrize("n", [1, 7, 4096, 1_000_003])
def test_add(capi, n):
    """Addition<3> on its own (opennn/addition_layer.h:65-76, y = a + b): bit for bit the fp32 sum, for sizes that are
    not a multiple of the vector width and for operands that start off a 16-byte boundary (the scalar path)."""
    rng = np.random.default_rng(n)
    a, b = rng.standard_normal(n + 1).astype(np.float32), rng.standard_normal(n + 1).astype(np.float32)
    for offset in (0, 1):
        a_d, b_d = dev(a)[offset:offset + n], dev(b)[offset:offset + n]
        out = capi.add(a_d, b_d)
        assert np.array_equal(host(out), a[offset:offset + n] + b[offset:offset + n])
    out = capi.add(dev(a)[:n], dev(a)[:n])                      # both operands the same buffer
    assert np.array_equal(host(out), a[:n] + a[:n])


@pytest.mark.parametrize("sms", [140, 132, 74, 3])
def test_sm_limit_keeps_results(capi, sms):
    """onn_set_sm_limit makes the persistent kernels (tcgen05 GEMMs with their split tail wave and split-K, the fused
    attention core, the staged cross-entropy) occupy fewer SMs, e.g. to leave some to NCCL; the results stay the same
    up to the order of the split sums."""
    from oracle import opennn_oracle as O
    rng = np.random.default_rng(sms)
    M, N, K = 4864, 1024, 512                           # 76 tile pairs: a split tail wave on 74 pairs, none on fewer
    a, b = dev(rng.standard_normal((M, K))), dev(0.05 * rng.standard_normal((K, N)))
    x = dev(rng.standard_normal((2, 256, 128)))
    p = {n: dev(rng.uniform(-0.1, 0.1, (128, 128))) for n in ("Wq", "Wk", "Wv", "Wo")}
    p.update({n: dev(0.05 * rng.standard_normal(128)) for n in ("bq", "bk", "bv", "bo")})
    logits = (3.0 * rng.standard_normal((1, 300, 8000))).astype(np.float32)
    targets = rng.integers(1, 8000, size=(1, 300)).astype(np.float32)

    def run():
        c, dw = torch.zeros(M, N, device="cuda"), torch.zeros(K, N, device="cuda")
        capi.gemm(a, b, c, M, N, K, K, N, N, 0, 1)
        capi.gemm(a, c, dw, K, N, M, K, N, N, 1, 1, split_k=4)               # dW = A^T C, reduction split four ways
        y, ws = capi.mha_fwd(x, x, p, 2, True)
        _, _, gradient, _ = capi.ce3d(dev(logits), dev(targets))
        return [host(t) for t in (c, dw, y, gradient)]

    reference = run()
    capi.check(capi.lib().onn_set_sm_limit(sms))
    try:
        limited = run()
    finally:
        capi.check(capi.lib().onn_set_sm_limit(0))
    for got, expected, what in zip(limited, reference, ("product", "split-K product", "attention output", "loss gradient")):
        assert_close(got, expected, 1e-4, what)                 # split sums are added in another order
    assert capi.lib().onn_gemm_device_status() == 0


@pytest.mark.parametrize("sms", [0, 132, 6])
def test_dynamic_work_keeps_results(capi, sms):
    """onn_set_dynamic_work: the persistent kernels take their tiles from a per-launch counter in the order the CTAs ask
    instead of a fixed share per CTA (what the data-parallel trainer runs with, so that SMs held by NCCL do not make a
    launch wait for the shares of CTAs that start late).  Same tiles, other owners: results equal up to the order of the
    split sums, launch after launch (the counters must come back to zero), with a split tail wave, split-K, the batched
    one-CTA kernel, attention forward and backward, and LayerNorm, on all SMs and on a few."""
    rng = np.random.default_rng(11 + sms)
    M, N, K = 4864, 1024, 512                           # 76 tile pairs: a split tail wave on 74 pairs
    a, b = dev(rng.standard_normal((M, K))), dev(0.05 * rng.standard_normal((K, N)))
    B, H, S, E = 3, 4, 256, 256
    x, dy = dev(rng.standard_normal((B, S, E))), dev(rng.standard_normal((B, S, E)))
    p = {n: dev(rng.uniform(-0.1, 0.1, (E, E))) for n in ("Wq", "Wk", "Wv", "Wo")}
    p.update({n: dev(0.05 * rng.standard_normal(E)) for n in ("bq", "bk", "bv", "bo")})
    gamma, beta = dev(rng.standard_normal(E)), dev(rng.standard_normal(E))

    def run():
        c, dw = torch.zeros(M, N, device="cuda"), torch.zeros(K, N, device="cuda")
        capi.gemm(a, b, c, M, N, K, K, N, N, 0, 1)
        capi.gemm(a, c, dw, K, N, M, K, N, N, 1, 1, split_k=4)
        y, ws = capi.mha_fwd(x, x, p, H, True)
        grads, dxq, _ = capi.mha_bwd(x, x, p, H, True, ws, dy)
        normed, mean, inv_std, _ = capi.layernorm_fwd(x, gamma, beta)
        dx, dgamma, dbeta = capi.layernorm_bwd(dy, x, mean, inv_std, gamma)
        return [host(t) for t in (c, dw, y, dxq, grads["dWq"], grads["dWv"], normed, dx, dgamma)]

    names = ("product", "split-K product", "attention output", "attention input gradient", "dWq", "dWv", "LayerNorm", "LayerNorm dx", "dgamma")
    reference = run()
    capi.check(capi.lib().onn_set_sm_limit(sms))
    previous = capi.lib().onn_set_dynamic_work(1)
    try:
        for repeat in range(3):
            for got, expected, what in zip(run(), reference, names):
                assert_close(got, expected, 1e-4, f"{what}, run {repeat}")
    finally:
        capi.lib().onn_set_dynamic_work(previous)
        capi.check(capi.lib().onn_set_sm_limit(0))
    assert capi.lib().onn_gemm_device_status() == 0


def test_dynamic_work_under_contention(capi):
    """The point of handing tiles out by counter: with 16 SMs held by another kernel (a bounded stand-in for NCCL's CTAs) a
    two-CTA GEMM whose CTAs own fixed shares waits for the shares of the CTAs that could not start; by counter it loses
    about the held SMs' share.  The margin asked for is far inside what is measured (0.32 ms against 0.21 ms)."""
    import ctypes
    import os
    if os.environ.get("ONN_B200_DYNAMIC_WORK") is not None:
        pytest.skip("the environment pins the mode this test switches")
    L = capi.lib()
    M, N, K = 16384, 4096, 1024
    a, b, c = torch.randn(M, K, device="cuda"), torch.randn(N, K, device="cuda") / 32, torch.empty(M, N, device="cuda")
    side = torch.cuda.Stream()

    def timed(held):
        # the median of five: a stand-in that got its SMs late in one repeat must not decide the figure
        seen = []
        for _ in range(5):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if held:
                capi.check(L.onn_selftest_hold_sms(held, ctypes.c_int64(10_000_000), ctypes.c_void_p(side.cuda_stream)))
                torch.cuda._sleep(1_000_000)               # ~0.5 ms: the stand-in has its SMs before the timed launches start
            start.record()
            for _ in range(10):
                capi.gemm(a, b, c, M, N, K, K, K, N, 0, 0)
            stop.record()
            torch.cuda.synchronize()
            seen.append(start.elapsed_time(stop) / 10)
        return sorted(seen)[len(seen) // 2]

    capi.gemm(a, b, c, M, N, K, K, K, N, 0, 0)
    fixed_alone, fixed_held = timed(0), timed(16)
    previous = L.onn_set_dynamic_work(1)
    try:
        capi.gemm(a, b, c, M, N, K, K, K, N, 0, 0)
        counter_alone, counter_held = timed(0), timed(16)
    finally:
        L.onn_set_dynamic_work(previous)
    print(f"\n[contention] fixed shares {fixed_alone:.3f} -> {fixed_held:.3f} ms, by counter {counter_alone:.3f} -> {counter_held:.3f} ms")
    assert counter_held < 0.85 * fixed_held, "tiles by counter must not wait for CTAs that start late"
    assert counter_held < 1.25 * counter_alone and counter_alone < 1.08 * fixed_alone
    assert L.onn_gemm_device_status() == 0


def test_adam_and_norm(capi):
    from oracle import opennn_oracle as O
    rng = np.random.default_rng(7)
    n = 100003                                   # odd size: exercises the scalar tail
    p0 = rng.standard_normal(n).astype(np.float32)
    m0 = (0.01 * rng.standard_normal(n)).astype(np.float32)
    v0 = (0.001 * rng.random(n)).astype(np.float32)
    for g_scale in (0.1, 1e-4):                  # clip active / inactive
        g0 = (g_scale * rng.standard_normal(n)).astype(np.float32)
        p, m, v, g = dev(p0), dev(m0), dev(v0), dev(g0)
        sqnorm = capi.grad_sqnorm(g)
        assert abs(float(sqnorm.item()) - float(np.sum(g0.astype(np.float64) ** 2))) <= 1e-5 * float(np.sum(g0.astype(np.float64) ** 2))
        capi.adam(p, m, v, g, 3, sqnorm=sqnorm, zero_grad=True)
        pe, me, ve = p0.copy(), m0.copy(), v0.copy()
        O.adam_update(pe, g0, me, ve, 3)
        assert_close(host(m), me, 1e-5, "m")
        assert_close(host(v), ve, 1e-5, "v")
        assert_close(host(p) - p0, pe - p0, 1e-4, "parameter update")
        assert not host(g).any(), "zero_grad must clear the gradient"


@pytest.mark.parametrize("V", [37, 4096, 32000])
def test_greedy_next_token_from_logits(capi, V):
    """Softmax and arg-max in one kernel give the token of the two separate kernels, on rows with exact ties, with
    logits so close that their probabilities round to the same float, and with a finished row."""
    rng = np.random.default_rng(V + 1)
    B, S = 7, 4
    x = rng.standard_normal((B, V)).astype(np.float32)
    x[1, 5] = x[1, V - 3] = 9.0                               # exact tie: the first index
    x[2, V // 2] = 8.0; x[2, 3] = np.nextafter(np.float32(8.0), np.float32(0))      # one ulp below, earlier in the row
    x[3] = 0.0                                                # a flat row
    x[4, V - 1] = 30.0                                        # saturated
    logits = dev(x)
    ids_a, ids_b = torch.zeros(B, S, device="cuda"), torch.zeros(B, S, device="cuda")
    fin_a = torch.zeros(B, dtype=torch.int32, device="cuda"); fin_a[6] = 1
    fin_b = fin_a.clone()
    capi.greedy_next_token_logits(logits, ids_a, fin_a, 1, end_id=V - 1)
    assert np.array_equal(host(logits), x), "the logits stay as they were"
    probabilities = capi.softmax_rows(logits.clone())
    capi.greedy_next_token_rows(probabilities, ids_b, fin_b, 1, end_id=V - 1)
    assert torch.equal(ids_a, ids_b) and torch.equal(fin_a, fin_b)
    assert host(ids_a)[1, 1] == 5 and host(ids_a)[3, 1] == 0 and host(ids_a)[4, 1] == V - 1 and host(fin_a)[4] == 1


@pytest.mark.parametrize("rows,features,out", [(6, 24, 1), (100, 64, 12), (300, 256, 128)])
def test_dense_sigmoid(capi, gemm_mode, rows, features, out):
    """Dense "Sigmoid" forward and backward against an fp64 evaluation: y = 1 / (1 + exp(-(x W + b))),
    delta = dY y (1 - y) written over dY, dW = X^T delta, db = column sums, dX = delta W^T."""
    rng = np.random.default_rng(rows + out)
    x = dev(rng.standard_normal((rows, features)).astype(np.float32))
    w = dev((0.2 * rng.standard_normal((features, out))).astype(np.float32))
    b = dev(rng.standard_normal(out).astype(np.float32))
    d_y = dev(rng.standard_normal((rows, out)).astype(np.float32))
    def close(a, e, what):
        # tf32 products: a single element may sit a little above 1e-3 of the largest; the L2 error may not
        max_err, l2_err = errors(host(a), host(e))
        assert l2_err <= TOL and max_err <= (2 * TOL if gemm_mode == "auto" else TOL), f"{what}: max {max_err:.2e}, l2 {l2_err:.2e}"

    y = capi.dense_fwd(x, w, b, "Sigmoid")
    expected_y = torch.sigmoid(x.double() @ w.double() + b.double())
    close(y, expected_y, "y")
    dx, dw, db = capi.dense_bwd(x, w, y, d_y.clone(), "Sigmoid")
    delta = d_y.double() * expected_y * (1 - expected_y)
    close(dw, x.double().t() @ delta, "dW")
    close(db, delta.sum(dim=0), "db")
    close(dx, delta @ w.double().t(), "dX")


@pytest.mark.parametrize("rows,features,out", [(8, 1024, 1024), (40, 256, 512), (3, 36, 20), (100, 64, 64)])
def test_dense_fwd_shared_input(capi, gemm_mode, rows, features, out):
    """Three Linear projections of one input in one call, two of them written into rows of a wider buffer (cache
    slots), against an fp64 product and against the three separate Dense forward passes (to rounding: the split of K
    may differ between one and three products per launch).  100 rows: one product after the other on the large-GEMM
    path.  Columns of the wider buffers past `out` stay untouched."""
    rng = np.random.default_rng(rows + out)
    x = dev(rng.standard_normal((rows, features)).astype(np.float32))
    weights = [dev((0.1 * rng.standard_normal((features, out))).astype(np.float32)) for _ in range(3)]
    biases = [dev(rng.standard_normal(out).astype(np.float32)) for _ in range(3)]
    pitches = [out, 5 * out, 3 * out + 4]
    outputs = [torch.full((rows, p), 7.0, device="cuda") for p in pitches]
    capi.dense_fwd_shared_input(x, weights, biases, outputs, pitches)
    for w, b, y in zip(weights, biases, outputs):
        separate = capi.dense_fwd(x, w, b, "Linear")
        assert_close(host(y[:, :out]), host(x.double() @ w.double() + b.double()), TOL, "product")
        assert_close(host(y[:, :out]), host(separate), 1e-5 if rows <= 16 or gemm_mode == "simt" else TOL, "against the separate pass")
        assert y.shape[1] == out or float((y[:, out:] - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("B,S_cache,length,E,H", [(3, 256, 256, 1024, 16), (2, 40, 17, 64, 8), (5, 9, 1, 32, 8), (2, 12, 12, 12, 2),
                                                  (1, 300, 299, 512, 2)])
def test_decode_attention(capi, B, S_cache, length, E, H):
    """Attention of one query row over cached keys and values against an fp64 evaluation: padded keys take the score
    -1e9 (a row of nothing but padding becomes uniform), slots past `length` are never read (they hold NaN here).
    Head sizes 64, 8, 4, 6 (not a multiple of 4: the one-warp kernel) and 256."""
    rng = np.random.default_rng(B * 100 + E)
    hd = E // H
    q = dev(rng.standard_normal((B, E)).astype(np.float32))
    k = dev(rng.standard_normal((B, S_cache, E)).astype(np.float32))
    v = dev(rng.standard_normal((B, S_cache, E)).astype(np.float32))
    k[:, length:] = float("nan"); v[:, length:] = float("nan")
    pad = torch.zeros(B, S_cache, dtype=torch.uint8, device="cuda")
    pad[0, length // 2:] = 1
    if B > 1:
        pad[1, :] = 1
    out = capi.decode_attention(q, k, v, pad, length, H)
    qh = q.double().view(B, H, 1, hd)
    kh = k[:, :length].double().view(B, length, H, hd).permute(0, 2, 1, 3)
    vh = v[:, :length].double().view(B, length, H, hd).permute(0, 2, 1, 3)
    scores = (qh @ kh.transpose(-1, -2)) / np.sqrt(hd)
    scores = torch.where(pad[:, None, None, :length].bool(), torch.full_like(scores, -1e9), scores)
    expected = (torch.softmax(scores, dim=-1) @ vh).reshape(B, E)
    assert_close(host(out), host(expected), 2e-5, "context")
    assert torch.equal(out, capi.decode_attention(q, k, v, pad, length, H)), "same bits on every run"
    assert torch.equal(out, capi.decode_attention(q, k, v, pad.t().contiguous(), length, H, position_major=True)), "flags stored per position"
    assert_close(host(capi.decode_attention(q, k, v, None, length, H)),
                 host((torch.softmax((qh @ kh.transpose(-1, -2)) / np.sqrt(hd), dim=-1) @ vh).reshape(B, E)), 2e-5, "no padding flags")


@pytest.mark.parametrize("V", [37, 4096, 32000, 32003])
def test_greedy_next_token_rows(capi, V):
    """Arg-max per row with the first index on ties, END marks a row finished, finished rows are left alone."""
    rng = np.random.default_rng(V)
    B, S = 6, 5
    p = rng.random((B, V)).astype(np.float32) * 0.5
    winners = [V - 1, 0, V // 2, 3, 7, V - 2]
    for b, w in enumerate(winners):
        p[b, w] = 0.9
    p[2, V // 2 + 5:V // 2 + 9] = 0.9                     # ties behind the winner: the first index wins
    if V > 2000:
        p[3, 3 + 1024] = 0.9                              # a tie held by another thread of the scan
    ids = torch.zeros(B, S, device="cuda")
    finished = torch.zeros(B, dtype=torch.int32, device="cuda")
    finished[4] = 1
    view = dev(p) if V % 4 == 0 else dev(np.concatenate([np.zeros((1, 1), np.float32), p.reshape(1, -1)], axis=1)).view(-1)[1:].view(B, V)
    capi.greedy_next_token_rows(view, ids, finished, 2, end_id=V - 2)
    got = host(ids)[:, 2]
    assert got.tolist() == [V - 1, 0, V // 2, 3, 0, V - 2]
    assert host(finished).tolist() == [0, 0, 0, 0, 1, 1]
    assert not host(ids)[:, [0, 1, 3, 4]].any()


@pytest.mark.parametrize("shape", [(1, 1024, 1024), (8, 4096, 1024), (13, 100, 36), (16, 32000, 256), (33, 1024, 4096),
                                   (64, 1024, 1024), (64, 40, 8), (20, 2048, 512), (30, 200, 72), (5, 64, 4096), (48, 520, 200), (17, 32000, 64)])
def test_gemm_few_rows(capi, shape):
    """At most 64 rows against a row-major [K, N] matrix (one decoding step): the cluster kernels that stream the matrix
    in column strips with K split over the CTAs of a cluster.  Ragged M, N and K, row pitches wider than the rows,
    bias + ReLU + alpha, accumulation into C, the same bits on every run.  fp32 arithmetic (1e-5) up to 16 rows or for
    a narrow matrix; tf32 operands with fp32 accumulation (1e-3) for 17 to 64 rows against at least 512 columns."""
    M, N, K = shape
    rng = np.random.default_rng(M * 7 + N + K)
    lda, ldb, ldc = K + 4, N + 8, N + 12
    A = torch.zeros(M, lda, device="cuda"); A[:, :K] = dev(rng.standard_normal((M, K)).astype(np.float32))
    W = torch.zeros(K, ldb, device="cuda"); W[:, :N] = dev(rng.standard_normal((K, N)).astype(np.float32))
    bias = dev(rng.standard_normal(N).astype(np.float32))
    product = A[:, :K].double() @ W[:, :N].double()
    capi.check(capi.lib().onn_gemm_set_mode(0))
    tol = 1e-3 if (M > 16 and N >= 512) else 1e-5

    out = torch.full((M, ldc), 7.0, device="cuda")
    capi.gemm(A, W, out, M, N, K, lda, ldb, ldc, 0, 1)
    assert_close(host(out[:, :N]), host(product), tol, "plain")
    assert float((out[:, N:] - 7.0).abs().max()) == 0.0, "columns past N must stay untouched"
    again = torch.full((M, ldc), 7.0, device="cuda")
    capi.gemm(A, W, again, M, N, K, lda, ldb, ldc, 0, 1)
    assert torch.equal(out, again), "the reduction over K must not depend on timing"

    capi.gemm(A, W, out, M, N, K, lda, ldb, ldc, 0, 1, bias=bias, relu=True, alpha=0.5)
    assert_close(host(out[:, :N]), host(torch.relu(0.5 * product + bias.double())), tol, "bias + ReLU + alpha")

    before = out.clone()
    capi.gemm(A, W, out, M, N, K, lda, ldb, ldc, 0, 1, flags=capi.ACCUMULATE)
    assert_close(host(out[:, :N]), host(before[:, :N].double() + product), tol, "accumulate")
    assert capi.lib().onn_gemm_device_status() == 0


@pytest.mark.parametrize("a_major,b_major", [(0, 1), (0, 0), (1, 1)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (300, 520, 136), (64, 48, 1056), (1000, 72, 40),
                                   (1000, 520, 136), (1024, 512, 200)])   # the last two reach the two-CTA kernel
def test_gemm_layouts(capi, gemm_mode, a_major, b_major, shape):
    """The GEMM primitive in every operand layout the layers use, with ragged M, N and K
    (zero-filled TMA boxes, masked epilogue) and each epilogue option."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    mask = rng.standard_normal((M, N)).astype(np.float32)
    A_store = dev(A if a_major == 0 else A.T)
    B_store = dev(B.T if b_major == 0 else B)
    lda = K if a_major == 0 else M
    ldb = K if b_major == 0 else N
    reference = A.astype(np.float64) @ B.astype(np.float64)

    out = torch.zeros(M, N, device="cuda")
    capi.gemm(A_store, B_store, out, M, N, K, lda, ldb, N, a_major, b_major)
    assert_close(host(out), reference, TOL, "plain")

    out = torch.zeros(M, N, device="cuda")
    sums = torch.ones(N, device="cuda")
    capi.gemm(A_store, B_store, out, M, N, K, lda, ldb, N, a_major, b_major, bias=dev(bias), relu=True, alpha=0.5, colsum_out=sums)
    expected = np.maximum(0.5 * reference + bias, 0)
    assert_close(host(out), expected, TOL, "alpha + bias + relu")
    assert_close(host(sums), 1.0 + expected.sum(axis=0), TOL, "column sums of the written values")

    start = rng.standard_normal((M, N)).astype(np.float32)
    out = dev(start)
    capi.gemm(A_store, B_store, out, M, N, K, lda, ldb, N, a_major, b_major, relu_mask=dev(mask), flags=capi.ACCUMULATE)
    assert_close(host(out), start + reference * (mask > 0), TOL, "mask + accumulate")

    out = dev(start)
    capi.gemm(A_store, B_store, out, M, N, K, lda, ldb, N, a_major, b_major, split_k=5)
    assert_close(host(out), start + reference, TOL, "split-K")

    # the ReLU mask as one bit per element: written by a ReLU GEMM for its own result, applied by another GEMM
    words = (N + 31) // 32
    bits = torch.full((M, words), -1, dtype=torch.int32, device="cuda")
    out = torch.zeros(M, N, device="cuda")
    capi.gemm(A_store, B_store, out, M, N, K, lda, ldb, N, a_major, b_major, bias=dev(bias), relu=True, relu_bits_out=bits, relu_bits_ld=words)
    written = host(out)
    positive = np.zeros((M, words * 32), dtype=bool)
    positive[:, :N] = written > 0
    expected_bits = (positive.reshape(M, words, 32).astype(np.uint64) << np.arange(32, dtype=np.uint64)).sum(axis=2).astype(np.uint32)
    valid = np.full((M, words), 0xFFFFFFFF, dtype=np.uint32)
    if N % 32: valid[:, -1] = (1 << (N % 32)) - 1            # bits past column N are unspecified
    got_bits = bits.cpu().numpy().view(np.uint32)
    assert np.array_equal(got_bits & valid, expected_bits & valid), "bits must equal (stored value > 0)"

    out = dev(start)
    sums = torch.zeros(N, device="cuda")
    capi.gemm(A_store, B_store, out, M, N, K, lda, ldb, N, a_major, b_major, relu_bits=bits, relu_bits_ld=words, colsum_out=sums)
    expected = reference * (written > 0)
    assert_close(host(out), expected, TOL, "bit mask")
    assert_close(host(sums), expected.sum(axis=0), TOL, "column sums after the bit mask", floor=1e-3 * np.abs(expected).sum(axis=0).max())


@pytest.mark.parametrize("B,H,Sq,Sk,causal,cross", [(2, 2, 256, 256, True, False), (2, 2, 256, 256, False, True),
                                                      (1, 3, 200, 136, False, True), (3, 1, 40, 72, False, True),
                                                      (2, 2, 72, 72, True, False),
                                                      # source lengths above 256: the kernels that walk the keys in tiles of 256
                                                      (2, 2, 300, 300, True, False), (1, 2, 130, 520, False, True),
                                                      (3, 1, 72, 260, False, True), (1, 2, 1024, 1024, True, False),
                                                      (2, 1, 512, 512, False, False), (2, 1, 384, 768, False, True)])
def test_mha_head64(capi, gemm_mode, B, H, Sq, Sk, causal, cross):
    """MultiHeadAttention at head size 64, the shapes the fused attention-core kernels serve (whole and ragged
    query tiles; source lengths up to 256 in one accumulator row, longer ones in key tiles of 256 with whole tiles
    above the causal diagonal skipped and a last tile of 4 keys; causal and key-padding masks), forward and backward
    against the oracle."""
    mha_head64_case(capi, gemm_mode, B, H, Sq, Sk, causal, cross)


@pytest.mark.parametrize("B,H,Sq,Sk,causal,cross", [(2, 2, 256, 256, True, False), (2, 2, 256, 256, False, True),
                                                      (1, 3, 200, 136, False, True), (3, 1, 40, 72, False, True),
                                                      (2, 2, 72, 72, True, False), (5, 16, 192, 192, True, False)])
def test_mha_head64_kv_grad_by_recomputation(capi, B, H, Sq, Sk, causal, cross):
    """The same layer with dK and dV from the kernel that forms the weights again on the SM (one key tile and two,
    ragged tiles, an item of a single query step, more work items than SMs), against the oracle."""
    previous = capi.lib().onn_mha_set_kv_grad_by_recomputation(1)
    try:
        launches = capi.lib().onn_launch_count()
        mha_head64_case(capi, "auto", B, H, Sq, Sk, causal, cross)
    finally:
        capi.lib().onn_mha_set_kv_grad_by_recomputation(previous)
    assert capi.lib().onn_launch_count() > launches


def mha_head64_case(capi, gemm_mode, B, H, Sq, Sk, causal, cross):
    from oracle import opennn_oracle as O
    E = 64 * H
    rng = np.random.default_rng(B * 1000 + Sq + Sk)
    limit = np.sqrt(6.0 / (2 * E))
    p = {n: rng.uniform(-limit, limit, (E, E)).astype(np.float32) for n in ("Wq", "Wk", "Wv", "Wo")}
    p.update({n: (0.05 * rng.standard_normal(E)).astype(np.float32) for n in ("bq", "bk", "bv", "bo")})
    xq = rng.standard_normal((B, Sq, E)).astype(np.float32)
    xs = rng.standard_normal((B, Sk, E)).astype(np.float32) if cross else xq
    if cross:
        xs[0, Sk - 5:] = 0.0                                  # padded source rows: masked keys
        if B > 1: xs[1, Sk // 2:] = 0.0
        if B > 2: xs[2, :] = 0.0                               # a source of nothing but padding: uniform weights
    delta = rng.standard_normal((B, Sq, E)).astype(np.float32)
    y_e, saved = O.mha_forward(xq, xs, p, H, causal)
    grads_e, dxq_e, dxs_e = O.mha_backward(xq, xs, p, H, saved, delta, not cross)

    pd = {k: dev(v) for k, v in p.items()}
    xq_d = dev(xq)
    xs_d = dev(xs) if cross else xq_d
    y, ws = capi.mha_fwd(xq_d, xs_d, pd, H, causal)
    weights = capi.mha_attention_weights(ws, B, Sq, Sk, E, H)
    # tf32 operands: the L2 error of every tensor stays within the tolerance; a single element of a reduction over
    # only 64 terms may exceed it (one product carries up to 9.8e-4), so the largest element error gets twice that
    def check(device, reference, what, floor=0.0):
        max_err, l2_err = errors(device, reference, floor)
        assert np.all(np.isfinite(device)), what
        if max_err > TOL:
            print(f"\n[mha_head64 B{B} H{H} Sq{Sq} Sk{Sk} causal{int(causal)} cross{int(cross)}] {what}: largest element error {max_err:.2e} (l2 {l2_err:.2e})")
        assert l2_err <= TOL and max_err <= (TOL if gemm_mode == "simt" else 2 * TOL), f"{what}: max-rel {max_err:.3e}, l2-rel {l2_err:.3e}"

    check(host(weights), saved["weights"], "attention weights")
    assert_close(host(weights).sum(axis=-1), np.ones((B, H, Sq)), 1e-3, "rows of the attention weights sum to one")
    check(host(y), y_e, "y")
    grads, dxq, dxs = capi.mha_bwd(xq_d, xs_d, pd, H, causal, ws, dev(delta))
    check(host(dxq), dxq_e, "dxq")
    if cross:
        check(host(dxs), dxs_e, "dxs")
    for name in ("dWq", "dWk", "dWv", "dWo", "dbq", "dbv", "dbo"):
        check(host(grads[name]), grads_e[name], name, floor=1e-6)
    # the key bias gradient is zero in exact arithmetic (a softmax row does not change when every score of the row
    # moves by the same amount), so it is compared on the scale of the query bias gradient
    assert np.abs(host(grads["dbk"]) - grads_e["dbk"]).max() <= 2 * TOL * max(np.abs(grads_e["dbq"]).max(), 1e-3), "dbk"
    assert capi.lib().onn_gemm_device_status() == 0


@pytest.mark.parametrize("a_major,b_major", [(0, 1), (0, 0), (1, 1)])
@pytest.mark.parametrize("M", [4864, 4800])
def test_gemm_split_tail_wave(capi, a_major, b_major, M):
    """76 tile pairs on 74 CTA pairs: the two tiles of the last wave are each split along the reduction between two
    pairs that ADD their halves into C, which the kernel zeroes first (or, with ONN_ACCUMULATE, adds to the caller's
    values).  Bias is added once, column sums see every element once, ragged M is clipped."""
    N, K = 1024, 1024
    rng = np.random.default_rng(M)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = (rng.standard_normal((K, N)) / 32).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    A_store = dev(A if a_major == 0 else A.T)
    B_store = dev(B.T if b_major == 0 else B)
    lda = K if a_major == 0 else M
    ldb = K if b_major == 0 else N
    reference = A.astype(np.float64) @ B.astype(np.float64)

    out = torch.full((M, N), 7.0, device="cuda")                 # stale values the kernel must not add to
    sums = torch.zeros(N, device="cuda")
    capi.gemm(A_store, B_store, out, M, N, K, lda, ldb, N, a_major, b_major, bias=dev(bias), alpha=0.5, colsum_out=sums)
    expected = 0.5 * reference + bias
    assert_close(host(out), expected, TOL, "alpha + bias over a split tail")
    assert_close(host(sums), expected.sum(axis=0), TOL, "column sums over a split tail", floor=1e-3 * np.abs(expected).sum(axis=0).max())

    start = rng.standard_normal((M, N)).astype(np.float32)
    out = dev(start)
    capi.gemm(A_store, B_store, out, M, N, K, lda, ldb, N, a_major, b_major, flags=capi.ACCUMULATE)
    assert_close(host(out), start + reference, TOL, "accumulate over a split tail")
    for _ in range(3):                                           # repeated launches take fresh tokens
        out2 = torch.full((M, N), -3.0, device="cuda")
        capi.gemm(A_store, B_store, out2, M, N, K, lda, ldb, N, a_major, b_major)
        assert_close(host(out2), reference, TOL, "plain product over a split tail")
    assert capi.lib().onn_gemm_device_status() == 0


@pytest.mark.parametrize("shape", [(1024, 512, 128), (300, 72, 40), (4864, 1024, 256)])
def test_gemm_reduction_through_operand_pairs(capi, gemm_mode, shape):
    """C = sum over p of A_p B_p^T for three operand pairs at equal distances (how dX = dQ Wq^T + dK Wk^T + dV Wv^T is
    computed): one launch of the two-CTA kernel where it applies, a store and two accumulating launches elsewhere."""
    M, N, K = shape
    rng = np.random.default_rng(M + N)
    a_gap, b_gap = M * K + 64, N * K + 8                        # the pairs need not be contiguous
    A = rng.standard_normal((3, M, K)).astype(np.float32)
    B = (rng.standard_normal((3, N, K)) / np.sqrt(3 * K)).astype(np.float32)
    A_store = torch.zeros(3 * a_gap, device="cuda")
    B_store = torch.zeros(3 * b_gap, device="cuda")
    for part in range(3):
        A_store[part * a_gap:part * a_gap + M * K] = dev(A[part]).reshape(-1)
        B_store[part * b_gap:part * b_gap + N * K] = dev(B[part]).reshape(-1)
    reference = sum(A[part].astype(np.float64) @ B[part].astype(np.float64).T for part in range(3))
    bias = rng.standard_normal(N).astype(np.float32)
    out = torch.full((M, N), 5.0, device="cuda")
    capi.gemm(A_store, B_store, out, M, N, K, K, K, N, 0, 0, bias=dev(bias), k_parts=3, part_strides=(a_gap, b_gap))
    assert_close(host(out), reference + bias, TOL, "three operand pairs")
    start = rng.standard_normal((M, N)).astype(np.float32)
    out = dev(start)
    capi.gemm(A_store, B_store, out, M, N, K, K, K, N, 0, 0, flags=capi.ACCUMULATE, k_parts=2, part_strides=(a_gap, b_gap))
    two = sum(A[part].astype(np.float64) @ B[part].astype(np.float64).T for part in range(2))
    assert_close(host(out), start + two, TOL, "two operand pairs, accumulated")
    assert capi.lib().onn_gemm_device_status() == 0


def test_gemm_batched_heads(capi, gemm_mode):
    """Per-(batch, head) products addressed by strides inside [B, S, E] tensors, as attention uses them."""
    Bn, H, Sq, Sk, hd = 3, 4, 40, 72, 16
    E = H * hd
    rng = np.random.default_rng(11)
    q = rng.standard_normal((Bn, Sq, E)).astype(np.float32)
    k = rng.standard_normal((Bn, Sk, E)).astype(np.float32)
    scores = torch.zeros(Bn, H, Sq, Sk, device="cuda")
    capi.gemm(dev(q), dev(k), scores, Sq, Sk, hd, E, E, Sk, 0, 0, alpha=0.25, batch_inner=H, batch_outer=Bn,
              a_strides=(hd, Sq * E), b_strides=(hd, Sk * E), c_strides=(Sq * Sk, H * Sq * Sk))
    qh = q.reshape(Bn, Sq, H, hd).transpose(0, 2, 1, 3).astype(np.float64)
    kh = k.reshape(Bn, Sk, H, hd).transpose(0, 2, 1, 3).astype(np.float64)
    assert_close(host(scores), 0.25 * qh @ kh.transpose(0, 1, 3, 2), TOL, "QK^T")
    p = rng.random((Bn, H, Sq, Sk)).astype(np.float32)
    ctx = torch.zeros(Bn, Sq, E, device="cuda")
    capi.gemm(dev(p), dev(k), ctx, Sq, hd, Sk, Sk, E, E, 0, 1, batch_inner=H, batch_outer=Bn,
              a_strides=(Sq * Sk, H * Sq * Sk), b_strides=(hd, Sk * E), c_strides=(hd, Sq * E))
    expected = (p.astype(np.float64) @ kh).transpose(0, 2, 1, 3).reshape(Bn, Sq, E)
    assert_close(host(ctx), expected, TOL, "PV")


def test_gemm_large_linearity(capi):
    """Full-size property check (config-5 FFN tile counts): C(A1 + A2) = C(A1) + C(A2) and a
    checksum against fp64 on sampled rows, on the tcgen05 path."""
    M, N, K = 8192, 4096, 1024
    gen = torch.Generator(device="cuda").manual_seed(3)
    A1 = torch.randn(M, K, device="cuda", generator=gen)
    A2 = torch.randn(M, K, device="cuda", generator=gen)
    W = torch.randn(K, N, device="cuda", generator=gen) * 0.05
    outs = []
    for A in (A1, A2, A1 + A2):
        out = torch.empty(M, N, device="cuda")
        capi.gemm(A, W, out, M, N, K, K, N, N, 0, 1)
        outs.append(out)
    assert capi.lib().onn_gemm_device_status() == 0
    assert_close(host(outs[2][::97]), host((outs[0] + outs[1])[::97]), TOL, "linearity")
    rows = torch.arange(0, M, 511, device="cuda")
    expected = A1[rows].double() @ W.double()
    assert_close(host(outs[0][rows]), host(expected), TOL, "sampled rows vs fp64")


def test_bounded_wait_gives_up_and_reports(capi):
    """Failure detection without a fault: a wait on a barrier nothing signals runs out after its
    limit, the kernel returns, the status word reports it once, and the context keeps working."""
    import ctypes
    assert capi.lib().onn_gemm_device_status() == 0
    gave_up = ctypes.c_int(-1)
    capi.check(capi.lib().onn_selftest_bounded_wait(ctypes.byref(gave_up)))
    assert gave_up.value == 1
    assert capi.lib().onn_gemm_device_status() == -5        # ONN_ERR_DEVICE_TIMEOUT, then cleared
    assert capi.lib().onn_gemm_device_status() == 0
    a = torch.randn(256, 64, device="cuda")
    b = torch.randn(64, 256, device="cuda")
    out = torch.empty(256, 256, device="cuda")
    capi.gemm(a, b, out, 256, 256, 64, 64, 256, 256, 0, 1)
    assert_close(host(out), host(a).astype(np.float64) @ host(b).astype(np.float64), TOL, "GEMM after the self-test")
