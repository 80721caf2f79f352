"""Generates the golden fixtures in this directory by running the UNMODIFIED reference CPU
library (oracle/_ref/onn_ref_harness, built by `make -C oracle` from an OpenNN checkout)
on seeded inputs.  The numpy restatement (oracle/opennn_oracle.py) is checked against every
output while the fixtures are written, so a fixture is only ever saved next to an oracle
that already agrees with the reference.

    python tests/golden/make_golden.py            # small cases (seconds)
    python tests/golden/make_golden.py --large    # + full-size configs 3, 4 and a batch-8 config 5 (minutes)

Fixtures are .npz files: inputs that cannot be regenerated cheaply, reference outputs, and
for the large configs per-view gradient norms plus strided samples instead of whole arenas.
Synthetic inputs stand in for a corpus: ids uniform in [1,V), seeded row lengths, right
padding with id 0.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import opennn_oracle as O  # noqa: E402
from oracle import ref_runner          # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
F32 = np.float32


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    denom = max(np.abs(b).max(), 1e-30)
    return float(np.abs(a - b).max() / denom)


def check(name, a, b, tol):
    e = rel_err(a, b)
    status = "ok" if e <= tol else "MISMATCH"
    print(f"    {name:28s} max|a-b|/max|b| = {e:.3e}  {status}")
    if e > tol:
        raise SystemExit(f"oracle disagrees with the reference on {name}")


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"  wrote {os.path.relpath(path, ROOT)} ({os.path.getsize(path) / 1024:.0f} KiB)")


def glorot(rng, shape, fan_in, fan_out):
    """The reference's Glorot-uniform: limit = sqrt(6/(inputs_number+outputs_number)) (layer.cpp:214-225)."""
    limit = np.sqrt(6.0 / (fan_in + fan_out))
    return rng.uniform(-limit, limit, shape).astype(F32)


# ---------------------------------------------------------------------------------------
# single layers (the shapes of the reference's own layer tests, plus config 1)
# ---------------------------------------------------------------------------------------

MHA_CASES = [
    # name, B, Sq, Sk, E, H, causal, cross, pad_rows
    ("mha_self_2_5_16_4", 2, 5, 5, 16, 4, 0, 0, 0),
    ("mha_causal_3_6_32_8", 3, 6, 6, 32, 8, 1, 0, 0),
    ("mha_cross_2_4_7_12_3", 2, 4, 7, 12, 3, 0, 1, 0),
    ("mha_self_8_3_8_2", 8, 3, 3, 8, 2, 0, 0, 0),
    ("mha_config1_8_16_32_4", 8, 16, 16, 32, 4, 0, 0, 0),
    ("mha_causal_pad_4_12_24_3", 4, 12, 12, 24, 3, 1, 0, 3),
    ("mha_cross_pad_3_9_14_64_4", 3, 9, 14, 64, 4, 0, 1, 4),
    ("mha_causal_2_40_128_2", 2, 40, 40, 128, 2, 1, 0, 5),
]


def mha_arena(p, E):
    parts = []
    for name in ("Wq", "bq", "Wk", "bk", "Wv", "bv", "Wo", "bo"):
        flat = p[name].ravel()
        slot = np.zeros(O.padded(flat.size), dtype=F32)
        slot[:flat.size] = flat
        parts.append(slot)
    return np.concatenate(parts)


def mha_unpack(arena, E):
    out, offset = {}, 0
    for name, shape in (("Wq", (E, E)), ("bq", (E,)), ("Wk", (E, E)), ("bk", (E,)),
                        ("Wv", (E, E)), ("bv", (E,)), ("Wo", (E, E)), ("bo", (E,))):
        count = int(np.prod(shape))
        out[name] = arena[offset:offset + count].reshape(shape)
        offset += O.padded(count)
    return out


def make_mha(seed=0):
    for name, B, Sq, Sk, E, H, causal, cross, pad_rows in MHA_CASES:
        print(f"  {name}")
        rng = np.random.default_rng(seed)
        p = {}
        for w, b in (("Wq", "bq"), ("Wk", "bk"), ("Wv", "bv"), ("Wo", "bo")):
            # MHA's inputs_number and outputs_number are both S*E (layer.cpp:214-225); applied to biases too
            p[w] = glorot(rng, (E, E), Sq * E, Sq * E) * F32(2.5)
            p[b] = glorot(rng, (E,), Sq * E, Sq * E) * F32(2.5)
        xq = rng.standard_normal((B, Sq, E)).astype(F32)
        xs = rng.standard_normal((B, Sk, E)).astype(F32) if cross else xq
        if pad_rows:
            # trailing source rows exactly zero -> key-padding mask fires (never row 0)
            (xs if cross else xq)[:, -pad_rows:, :] = 0
        delta = rng.standard_normal((B, Sq, E)).astype(F32)
        arena = mha_arena(p, E)
        tensors = {"params": arena, "x0": xq, "delta": delta}
        if cross:
            tensors["x1"] = xs
        spec = dict(mode="layer", kind="mha", B=B, S=Sq, Sk=Sk, E=E, H=H, causal=causal, cross=cross)
        ref, _ = ref_runner.run(spec, tensors, ["y", "attention_weights", "grads", "dx0", "dx1"])
        y, saved = O.mha_forward(xq, xs, p, H, bool(causal))
        g, dxq, dxs = O.mha_backward(xq, xs, p, H, saved, delta, not cross)
        check("y", y, ref["y"], 2e-5)
        check("attention_weights", saved["weights"], ref["attention_weights"], 2e-5)
        check("grads", mha_arena({k[1:]: v for k, v in g.items()}, E), ref["grads"], 5e-5)
        check("dx0", dxq, ref["dx0"], 5e-5)
        out = dict(spec=np.array([B, Sq, Sk, E, H, causal, cross]), params=arena, xq=xq, delta=delta,
                   y=ref["y"], attention_weights=ref["attention_weights"], grads=ref["grads"], dxq=ref["dx0"])
        if cross:
            check("dx1", dxs, ref["dx1"], 5e-5)
            out.update(xs=xs, dxs=ref["dx1"])
        save(name, **out)


EMBEDDING_CASES = [
    # name, B, S, V, E, scale, add_pe
    ("embedding_2_10_5_8", 2, 10, 5, 8, 1, 1),
    ("embedding_3_7_11_16_noscale", 3, 7, 11, 16, 0, 1),
    ("embedding_2_12_8_32_nope", 2, 12, 8, 32, 1, 0),
    ("embedding_4_33_50_20", 4, 33, 50, 20, 1, 1),
]


def make_embedding(seed=1):
    for name, B, S, V, E, scale, add_pe in EMBEDDING_CASES:
        print(f"  {name}")
        rng = np.random.default_rng(seed)
        weights = (F32(0.05) * rng.uniform(-1, 1, (V, E))).astype(F32)   # row 0 deliberately NOT zero here
        ids = rng.integers(0, V, size=(B, S)).astype(F32)                # includes pad id 0
        ids[0, 1] = -3          # out of range below
        ids[1, 2] = V           # out of range above
        ids[1, 3] = V + 7
        ids[0, 4] = F32(2.75)   # truncates to 2
        delta = rng.standard_normal((B, S, E)).astype(F32)
        arena = np.zeros(O.padded(V * E), dtype=F32)
        arena[:V * E] = weights.ravel()
        spec = dict(mode="layer", kind="embedding", B=B, S=S, V=V, E=E, scale=scale, add_pe=add_pe)
        ref, _ = ref_runner.run(spec, {"params": arena, "x0": ids, "delta": delta}, ["y", "grads"])
        pe = O.positional_encoding(S, E)
        y = O.embedding_forward(ids, weights, pe, bool(scale), bool(add_pe))
        dW = O.embedding_backward(ids, delta, V, bool(scale))
        ref_y = ref["y"].reshape(B, S, E)
        if not np.array_equal(y.view(np.uint32), ref_y.view(np.uint32)):
            raise SystemExit("embedding forward is not bit-exact against the reference")
        print("    y                            bit-exact")
        check("dW", dW, ref["grads"][:V * E], 1e-6)
        save(name, spec=np.array([B, S, V, E, scale, add_pe]), weights=weights, ids=ids, delta=delta,
             pe=pe, y=ref_y, dW=ref["grads"][:V * E].reshape(V, E))


LAYERNORM_CASES = [("layernorm_2_5_8", 2, 5, 8), ("layernorm_4_10_16", 4, 10, 16),
                   ("layernorm_1_32_64", 1, 32, 64), ("layernorm_8_4_12", 8, 4, 12),
                   ("layernorm_3_7_512", 3, 7, 512), ("layernorm_2_9_1000", 2, 9, 1000)]


def make_layernorm(seed=2):
    for name, B, S, E in LAYERNORM_CASES:
        print(f"  {name}")
        rng = np.random.default_rng(seed)
        x = (5 * rng.standard_normal((B, S, E))).astype(F32)   # N(0,5) as in the reference's test
        gammas = rng.uniform(0.5, 1.5, E).astype(F32)
        betas = rng.uniform(-0.5, 0.5, E).astype(F32)
        delta = rng.standard_normal((B, S, E)).astype(F32)
        arena = np.zeros(2 * O.padded(E), dtype=F32)
        arena[:E] = gammas
        arena[O.padded(E):O.padded(E) + E] = betas
        spec = dict(mode="layer", kind="layernorm", B=B, S=S, E=E)
        ref, _ = ref_runner.run(spec, {"params": arena, "x0": x, "delta": delta}, ["y", "grads", "dx0"])
        y, mean, std, x_hat = O.layernorm_forward(x, gammas, betas)
        dx, dg, db = O.layernorm_backward(delta, x_hat, std, gammas)
        check("y", y, ref["y"], 1e-5)
        check("dx", dx, ref["dx0"], 2e-5)
        check("dgamma", dg, ref["grads"][:E], 2e-5)
        check("dbeta", db, ref["grads"][O.padded(E):O.padded(E) + E], 2e-5)
        save(name, spec=np.array([B, S, E]), x=x, gammas=gammas, betas=betas, delta=delta,
             y=ref["y"], dx=ref["dx0"], dgamma=ref["grads"][:E], dbeta=ref["grads"][O.padded(E):O.padded(E) + E])


POOLING_CASES = [("pooling_max_3_7_16", 3, 7, 16, "MaxPooling"), ("pooling_max_2_33_200", 2, 33, 200, "MaxPooling"),
                 ("pooling_avg_4_9_24", 4, 9, 24, "AveragePooling"), ("pooling_avg_2_40_136", 2, 40, 136, "AveragePooling")]


def make_pooling(seed=6):
    for name, B, S, E, method in POOLING_CASES:
        print(f"  {name}")
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((B, S, E)).astype(F32)
        x[:, S - 2:, :] = 0                                       # trailing padding rows
        x[0, 1, :] = 0                                            # one in the middle
        if B > 2:
            x[2] = 0                                              # a sample of nothing but padding
        x[1, 0, 3] = x[1, 2, 3] = 7.5                             # a tie for the maximum: the first position wins
        delta = rng.standard_normal((B, E)).astype(F32)
        spec = dict(mode="layer", kind="pooling3d", B=B, S=S, E=E, method=method)
        ref, _ = ref_runner.run(spec, {"params": np.zeros(0, dtype=F32), "x0": x, "delta": delta}, ["y", "dx0"])
        y, saved = O.pooling3d_forward(x, method)
        dx = O.pooling3d_backward(x, delta, method, saved)
        check("y", y, ref["y"], 1e-6)
        check("dx", dx, ref["dx0"], 1e-6)
        save(name, spec=np.array([B, S, E]), method=np.array(method), x=x, delta=delta, y=ref["y"].reshape(B, E), dx=ref["dx0"].reshape(B, S, E))


CLASSIFIER_CASES = {
    # name: B, S, V, E, H, hidden, classes, steps
    "classifier_tiny": (6, 12, 50, 16, 2, 24, 3, 3),
    "classifier_head64": (8, 72, 200, 128, 2, 256, 5, 3),
    "classifier_binary": (6, 12, 50, 16, 2, 24, 1, 3),        # one output: Sigmoid + the binary cross-entropy
}


def classifier_inputs(name):
    """Seeded parameters, ids and one-hot targets of a classifier case (shared by the generator and the tests)."""
    B, S, V, E, H, hidden, classes, steps = CLASSIFIER_CASES[name]
    rng = np.random.default_rng(11 + B + S)
    net = O.build_text_classifier(V, S, E, H, [hidden], classes)
    params = net.default_parameters(rng)
    ids = O.synthetic_ids(rng, B, S, V, max(2, S // 3), S)
    labels = rng.integers(0, max(classes, 2), B)
    targets = np.eye(classes, dtype=F32)[labels] if classes > 1 else labels.astype(F32).reshape(B, 1)
    return net, params, ids, targets


def make_classifier():
    for name, (B, S, V, E, H, hidden, classes, steps) in CLASSIFIER_CASES.items():
        print(f"  {name}")
        net, params, ids, targets = classifier_inputs(name)
        spec = dict(mode="classifier", B=B, S=S, V=V, E=E, H=H, hidden=hidden, classes=classes, steps=steps)
        ref, _ = ref_runner.run(spec, {"params": params, "ids": ids, "targets": targets},
                                ["param_count", "grad_step0", "loss", "params_out", "probabilities"])
        assert int(ref["param_count"][0]) == net.parameters_size
        arena, m, v = params.copy(), np.zeros_like(params), np.zeros_like(params)
        iteration, losses = 1, []
        for step in range(steps):
            if step == 0:
                check("probabilities", net.forward(arena, {-1: ids}), ref["probabilities"], 1e-5)
            error, gradient, iteration = net.train_step_2d(arena, m, v, iteration, ids, targets)
            if step == 0:
                check("gradient", gradient, ref["grad_step0"], 1e-5)
            losses.append(error)
        check("loss history", np.array(losses), ref["loss"], 1e-6)
        check("params_out", arena, ref["params_out"], 1e-4)       # Adam turns rounding differences of tiny gradients into steps
        save(name, probabilities=ref["probabilities"].reshape(B, classes), gradient=ref["grad_step0"], loss=ref["loss"], params_out=ref["params_out"])


DENSE_CASES = [("dense_linear_2_5_6_9", 2, 5, 6, 9, "Linear"), ("dense_relu_3_8_16_40", 3, 8, 16, 40, "RectifiedLinear"),
               ("dense_softmax_4_5_6_8", 4, 5, 6, 8, "Softmax"), ("dense_relu_2_33_64_136", 2, 33, 64, 136, "RectifiedLinear"),
               ("dense_linear_2_17_200_72", 2, 17, 200, 72, "Linear")]


def make_dense(seed=3):
    for name, B, S, E, F, activation in DENSE_CASES:
        print(f"  {name}")
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((B, S, E)).astype(F32)
        weights = rng.uniform(-0.3, 0.3, (E, F)).astype(F32)
        biases = rng.uniform(-0.3, 0.3, F).astype(F32)
        delta = rng.standard_normal((B, S, F)).astype(F32)
        arena = np.zeros(O.padded(F) + O.padded(E * F), dtype=F32)
        arena[:F] = biases
        arena[O.padded(F):O.padded(F) + E * F] = weights.ravel()
        spec = dict(mode="layer", kind="dense", B=B, S=S, E=E, F=F, activation=activation)
        ref, _ = ref_runner.run(spec, {"params": arena, "x0": x, "delta": delta}, ["y", "grads", "dx0"])
        y, derivatives = O.dense_forward(x, weights, biases, activation)
        dx, dW, db = O.dense_backward(x, weights, delta, derivatives, activation)
        check("y", y, ref["y"], 1e-5)
        check("dx", dx, ref["dx0"], 1e-5)
        check("db", db, ref["grads"][:F], 1e-5)
        check("dW", dW, ref["grads"][O.padded(F):O.padded(F) + E * F], 1e-5)
        save(name, spec=np.array([B, S, E, F]), activation=np.array(activation), x=x, weights=weights, biases=biases,
             delta=delta, y=ref["y"], dx=ref["dx0"], db=ref["grads"][:F],
             dW=ref["grads"][O.padded(F):O.padded(F) + E * F])


CE_CASES = [("ce3d_4_5_8", 4, 5, 8), ("ce3d_3_11_1000", 3, 11, 1000), ("ce3d_2_6_37", 2, 6, 37)]


def make_ce3d(seed=4):
    for name, B, S, V in CE_CASES:
        print(f"  {name}")
        rng = np.random.default_rng(seed)
        logits = (3 * rng.standard_normal((B, S, V))).astype(F32)
        p = O.softmax_last(logits)
        targets = rng.integers(0, V, size=(B, S)).astype(F32)     # 0 = masked, as rand()%V in the reference test
        targets[0, 0] = 0
        targets[0, 1] = V       # out of range -> inactive
        targets[0, 2] = -2
        # make a few predictions correct so accuracy is not 0
        best = p.argmax(axis=-1)
        targets[1, :3] = best[1, :3]
        spec = dict(mode="ce3d", B=B, S=S, V=V)
        ref, _ = ref_runner.run(spec, {"p": p, "targets": targets}, ["loss", "dlogits"])
        error, accuracy, count = O.ce3d_error(p, targets)
        grad = O.ce3d_output_gradients(p, targets)
        check("error", [error], ref["loss"][:1], 1e-6)
        check("accuracy", [accuracy], ref["loss"][1:2], 1e-6)
        check("dlogits", grad, ref["dlogits"], 1e-6)
        save(name, spec=np.array([B, S, V]), logits=logits, p=p, targets=targets, loss=ref["loss"], dlogits=ref["dlogits"])


# ---------------------------------------------------------------------------------------
# whole networks
# ---------------------------------------------------------------------------------------

CONFIGS = {
    # name: (mode, B, S_in, S_dec, V_in, V_out, E, H, F, L, steps, seed, min_len, max_len)
    "config2_tiny": ("transformer", 32, 32, 32, 1000, 1000, 64, 4, 128, 1, 3, 0, 8, 32),
    "tiny_encdec_odd": ("transformer", 3, 11, 7, 50, 41, 24, 3, 40, 2, 2, 5, 3, 7),
    "tiny_decoder_only": ("decoder", 4, 0, 64, 0, 500, 64, 8, 128, 2, 3, 6, 64, 64),
    "config3_mid": ("transformer", 64, 128, 128, 8000, 8000, 512, 8, 2048, 6, 10, 1, 32, 128),
    "config4_long": ("decoder", 16, 0, 1024, 0, 8000, 512, 8, 2048, 2, 2, 2, 1024, 1024),
    "config5_batch8": ("transformer", 8, 256, 256, 32000, 32000, 1024, 16, 4096, 6, 1, 3, 64, 256),
}
LARGE = {"config3_mid", "config4_long", "config5_batch8"}


def network_inputs(name):
    """Seeded inputs of a CONFIGS entry: (network, parameter arena, external inputs, targets)."""
    mode, B, S_in, S_dec, V_in, V_out, E, H, F, L, steps, seed, lo, hi = CONFIGS[name]
    rng = np.random.default_rng(seed)
    if mode == "transformer":
        net = O.build_transformer(S_in, S_dec, V_in, V_out, E, H, F, L)
        enc = O.synthetic_ids(rng, B, S_in, V_in, min(lo, S_in), min(hi, S_in))
    else:
        net = O.build_decoder_only(S_dec, V_out, E, H, F, L)
        enc = None
    dec = O.synthetic_ids(rng, B, S_dec, V_out, min(lo, S_dec), min(hi, S_dec))
    targets = O.synthetic_ids(rng, B, S_dec, V_out, min(lo, S_dec), min(hi, S_dec))
    params = net.default_parameters(rng)
    external = {-1: dec} if enc is None else {-1: dec, -2: enc}
    return net, params, external, targets


def view_norms(net, arena):
    norms = []
    for layer in net.layers:
        for name, (offset, shape) in layer["views"].items():
            count = int(np.prod(shape))
            norms.append(np.sqrt(np.sum(arena[offset:offset + count].astype(np.float64) ** 2)))
    return np.array(norms)


def make_network(name):
    mode, B, S_in, S_dec, V_in, V_out, E, H, F, L, steps, seed, lo, hi = CONFIGS[name]
    print(f"  {name}")
    net, params, external, targets = network_inputs(name)
    small = name not in LARGE
    spec = dict(mode=mode, B=B, S_in=S_in, S_dec=S_dec, V_in=V_in, V_out=V_out, E=E, H=H, F=F, L=L,
                steps=steps, lr=1e-3, dump_layers=1 if small else 0)
    tensors = {"params": params, "dec_ids": external[-1], "targets": targets}
    if -2 in external:
        tensors["enc_ids"] = external[-2]
    wanted = ["loss", "grad_step0", "params_out", "param_count"]
    if small:
        wanted += [f"layer_out_{i}" for i in range(len(net.layers))]
    ref, seconds = ref_runner.run(spec, tensors, wanted)
    assert int(ref["param_count"][0]) == net.parameters_size, (ref["param_count"], net.parameters_size)
    print(f"    reference: {steps} steps, {np.mean(seconds):.2f} s/step; loss {ref['loss'][0::2]}")

    out = dict(loss=ref["loss"], grad_view_norms=view_norms(net, ref["grad_step0"]),
               grad_norm=np.array(np.sqrt(np.sum(ref["grad_step0"].astype(np.float64) ** 2))),
               ref_seconds_per_step=np.array(seconds))
    stride = 1 if small else 4099
    out["sample_stride"] = np.array(stride)
    out["grad_sample"] = ref["grad_step0"][::stride]
    out["params_out_sample"] = ref["params_out"][::stride]
    if small:
        last = ref[f"layer_out_{len(net.layers) - 1}"]
        out["last_layer_stride"] = np.array(1 if last.size < 100000 else 13)
        out["last_layer_out"] = last[::int(out["last_layer_stride"])]
        out["layer_out_norms"] = np.array([np.sqrt(np.sum(ref[f"layer_out_{i}"].astype(np.float64) ** 2))
                                           for i in range(len(net.layers))])

    # the numpy restatement must agree with the reference (the large configs would take too long in numpy)
    if small:
        arena = params.copy()
        m = np.zeros_like(arena)
        v = np.zeros_like(arena)
        iteration = 1
        losses = []
        for step in range(steps):
            error, accuracy, gradient, iteration = net.train_step(arena, m, v, iteration, external, targets)
            losses += [error, accuracy]
            if step == 0:
                for i in range(len(net.layers)):
                    check(f"layer_out_{i} ({net.layers[i]['kind']})", net.outputs[i], ref[f"layer_out_{i}"], 5e-5)
                check("grad_step0", gradient, ref["grad_step0"], 2e-4)
        check("loss history", losses[0::2], ref["loss"][0::2], 1e-5)
        check("accuracy history", np.array(losses[1::2]) + 1, ref["loss"][1::2] + 1, 1e-6)
        check("params_out", arena, ref["params_out"], 1e-4)
    save(name, **out)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--large", action="store_true")
    parser.add_argument("--only", default="")
    args = parser.parse_args()
    if not ref_runner.available():
        raise SystemExit("build the reference first: make -C oracle REF=/path/to/opennn")
    groups = {"mha": make_mha, "embedding": make_embedding, "layernorm": make_layernorm,
              "dense": make_dense, "ce3d": make_ce3d, "pooling": make_pooling,
              "classifier": make_classifier}
    for group, fn in groups.items():
        if args.only and args.only != group:
            continue
        print(group)
        fn()
    for name in CONFIGS:
        if args.only and args.only != name and args.only != "networks":
            continue
        if name in LARGE and not args.large:
            continue
        print("network")
        make_network(name)


if __name__ == "__main__":
    main()
