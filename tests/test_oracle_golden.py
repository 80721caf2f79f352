"""CPU: the numpy restatement (oracle/opennn_oracle.py) against the golden fixtures that the
unmodified reference CPU library produced (tests/golden/make_golden.py)."""

import glob
import os

import numpy as np
import pytest

from oracle import opennn_oracle as O
from tests.util import GOLDEN, assert_close, golden
from tests.golden.make_golden import CONFIGS, LARGE, mha_unpack, network_inputs, view_norms


def names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


@pytest.mark.parametrize("name", names("embedding_"))
def test_embedding_bit_exact(name):
    g = golden(name)
    B, S, V, E, scale, add_pe = g["spec"]
    pe = O.positional_encoding(int(S), int(E))
    assert np.array_equal(pe.view(np.uint32), g["pe"].view(np.uint32))
    y = O.embedding_forward(g["ids"], g["weights"], pe, bool(scale), bool(add_pe))
    assert np.array_equal(y.view(np.uint32), g["y"].view(np.uint32)), "embedding forward must match the reference bit for bit"
    dW = O.embedding_backward(g["ids"], g["delta"], int(V), bool(scale))
    assert_close(dW, g["dW"], 1e-6, "dW")
    assert not dW[0].any(), "padding row gradient must be exactly zero"


@pytest.mark.parametrize("name", names("layernorm_"))
def test_layernorm(name):
    g = golden(name)
    y, mean, std, x_hat = O.layernorm_forward(g["x"], g["gammas"], g["betas"])
    dx, dg, db = O.layernorm_backward(g["delta"], x_hat, std, g["gammas"])
    assert_close(y, g["y"], 1e-5, "y")
    assert_close(dx, g["dx"], 2e-5, "dx")
    assert_close(dg, g["dgamma"], 2e-5, "dgamma")
    assert_close(db, g["dbeta"], 2e-5, "dbeta")


@pytest.mark.parametrize("name", names("pooling_"))
def test_pooling3d(name):
    g = golden(name)
    method = str(g["method"])
    y, saved = O.pooling3d_forward(g["x"], method)
    dx = O.pooling3d_backward(g["x"], g["delta"], method, saved)
    assert np.array_equal(y, g["y"]) and np.array_equal(dx, g["dx"])


@pytest.mark.parametrize("name", names("dense_"))
def test_dense(name):
    g = golden(name)
    activation = str(g["activation"])
    y, derivatives = O.dense_forward(g["x"], g["weights"], g["biases"], activation)
    dx, dW, db = O.dense_backward(g["x"], g["weights"], g["delta"], derivatives, activation)
    assert_close(y, g["y"], 1e-5, "y")
    assert_close(dx, g["dx"], 1e-5, "dx")
    assert_close(dW, g["dW"], 1e-5, "dW")
    assert_close(db, g["db"], 1e-5, "db")


@pytest.mark.parametrize("name", names("mha_"))
def test_mha(name):
    g = golden(name)
    B, Sq, Sk, E, H, causal, cross = (int(v) for v in g["spec"])
    p = mha_unpack(g["params"], E)
    xs = g["xs"] if cross else g["xq"]
    y, saved = O.mha_forward(g["xq"], xs, p, H, bool(causal))
    grads, dxq, dxs = O.mha_backward(g["xq"], xs, p, H, saved, g["delta"], not cross)
    assert_close(y, g["y"], 2e-5, "y")
    assert_close(saved["weights"], g["attention_weights"], 2e-5, "attention weights")
    assert_close(dxq, g["dxq"], 5e-5, "dxq")
    if cross:
        assert_close(dxs, g["dxs"], 5e-5, "dxs")
    ref = mha_unpack(g["grads"], E)
    floor = float(np.abs(g["grads"]).max())
    for name_ in ref:
        assert_close(grads["d" + name_], ref[name_], 5e-5, "d" + name_, floor=floor)


@pytest.mark.parametrize("name", names("ce3d_"))
def test_ce3d(name):
    g = golden(name)
    error, accuracy, count = O.ce3d_error(g["p"], g["targets"])
    grad = O.ce3d_output_gradients(g["p"], g["targets"])
    assert abs(error - g["loss"][0]) <= 1e-6 * max(1.0, abs(g["loss"][0]))
    assert abs(accuracy - g["loss"][1]) <= 1e-6
    assert_close(grad, g["dlogits"], 1e-6, "dlogits")


@pytest.mark.parametrize("name", [n for n in CONFIGS if n not in LARGE])
def test_network_training_steps(name):
    """Forward, loss, backward and Adam for whole networks: loss history, first-step gradient,
    parameters after the last step."""
    g = golden(name)
    steps = CONFIGS[name][10]
    net, params, external, targets = network_inputs(name)
    arena, m, v, iteration = params.copy(), np.zeros_like(params), np.zeros_like(params), 1
    for step in range(steps):
        error, accuracy, gradient, iteration = net.train_step(arena, m, v, iteration, external, targets)
        assert abs(error - g["loss"][2 * step]) <= 1e-5 * abs(g["loss"][2 * step])
        assert abs(accuracy - g["loss"][2 * step + 1]) <= 1e-6
        if step == 0:
            assert_close(gradient, g["grad_sample"], 2e-4, "gradient")
            assert_close(view_norms(net, gradient), g["grad_view_norms"], 1e-4, "per-view gradient norms")
            stride = int(g["last_layer_stride"])
            assert_close(net.outputs[-1].ravel()[::stride], g["last_layer_out"], 5e-5, "probabilities")
    assert_close(arena, g["params_out_sample"], 1e-4, "parameters after Adam")


@pytest.mark.parametrize("name", sorted(LARGE))
def test_full_size_network_first_step(name):
    """The restatement at the full size of configs 3, 4 and a batch-8 slice of config 5 against what the reference
    left in the fixtures: first-step loss and accuracy, per-view gradient norms, every 4099th gradient element.  The
    GPU parity tests judge whole gradient arenas at these sizes with this restatement, so it is pinned here first.
    Two fp32 evaluations with different summation orders (Eigen there, BLAS here) already put a few ReLU
    pre-activations on opposite sides of zero at this size, which shows as 4e-4 to 6e-4 in the sampled gradient
    (2e-4 bounds the small networks); loss, accuracy and the per-view norms are not sensitive to it."""
    g = golden(name)
    net, params, external, targets = network_inputs(name)
    probabilities = net.forward(params, external)
    error, accuracy, _ = O.ce3d_error(probabilities, targets)
    assert abs(error - g["loss"][0]) <= 1e-5 * abs(g["loss"][0])
    assert abs(accuracy - g["loss"][1]) <= 1e-6
    gradient = net.backward(params, O.ce3d_output_gradients(probabilities, targets))
    assert_close(gradient[::int(g["sample_stride"])], g["grad_sample"], 1e-3, "gradient samples")
    assert_close(view_norms(net, gradient), g["grad_view_norms"], 2e-4, "per-view gradient norms")


@pytest.mark.parametrize("name", ["classifier_tiny", "classifier_head64", "classifier_binary"])
def test_text_classifier_training_steps(name):
    """Embedding -> attention -> max pooling -> Dense<2> head with the 2-D cross-entropy, against the reference's
    probabilities, first gradient, loss history and parameters after three Adam steps."""
    from tests.golden.make_golden import CLASSIFIER_CASES, classifier_inputs
    g = golden(name)
    steps = CLASSIFIER_CASES[name][-1]
    net, params, ids, targets = classifier_inputs(name)
    arena, m, v = params.copy(), np.zeros_like(params), np.zeros_like(params)
    assert_close(net.forward(arena, {-1: ids}), g["probabilities"], 1e-5, "probabilities")
    iteration, losses = 1, []
    for step in range(steps):
        error, gradient, iteration = net.train_step_2d(arena, m, v, iteration, ids, targets)
        if step == 0:
            assert_close(gradient, g["gradient"], 1e-5, "gradient")
        losses.append(error)
    assert_close(np.array(losses), g["loss"], 1e-6, "loss history")
    assert_close(arena, g["params_out"], 1e-4, "parameters after Adam")


def test_transformer_structure():
    """Layer count and order of the reference's Transformer builder: 2 + 7L + 10L + 1 layers
    (20 for L = 1, the figure the reference's own structural test checks)."""
    net = O.build_transformer(32, 32, 1000, 1000, 64, 4, 128, 1)
    assert len(net.layers) == 20
    assert net.parameters_size == 276712
    kinds = [l["kind"] for l in net.layers]
    assert kinds[:2] == ["Embedding", "Embedding"]
    assert kinds[2:9] == ["MultiHeadAttention", "Addition3d", "Normalization3d", "Dense3d", "Dense3d", "Addition3d", "Normalization3d"]
    assert kinds[-1] == "Dense3d" and net.layers[-1]["activation"] == "Softmax"
    assert net.layers[0]["inputs"] == [-1] and net.layers[1]["inputs"] == [-2]
    assert net.layers[12]["inputs"] == [11, 8], "cross-attention reads the decoder norm and the encoder output"


def test_adam_first_step_uses_iteration_two():
    rng = np.random.default_rng(0)
    p = rng.standard_normal(64).astype(np.float32)
    g = (0.01 * rng.standard_normal(64)).astype(np.float32)
    m, v = np.zeros_like(p), np.zeros_like(p)
    before = p.copy()
    O.adam_update(p, g, m, v, 2, lr=1e-3)
    bc1, bc2 = 1 - 0.9 ** 2, 1 - 0.999 ** 2
    expected = before - 1e-3 * ((0.1 * g) / bc1) / (np.sqrt(0.001 * g * g / bc2) + np.finfo(np.float32).eps)
    assert np.allclose(p, expected, rtol=1e-5, atol=1e-7)
