"""CPU restatement (numpy, fp32) of OpenNN's transformer training path.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA path: only the tests,
the smoke check and the benchmark's CPU-baseline leg may import it.  No product code does.

Parity is pinned: `tests/golden/make_golden.py` runs the unmodified reference CPU library
(built by `oracle/Makefile` into `oracle/_ref/`) on the same seeded inputs and compares
every function below with it; the outputs it produced are committed under `tests/golden/`.

Each function cites the reference file:line (paths inside the OpenNN checkout) it follows.
All arithmetic is float32 unless the reference itself uses double.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32
EPSILON = np.finfo(np.float32).eps  # opennn/pch.h:123  numeric_limits<float>::epsilon()


def _mm(a, b):
    """Every contraction of the path goes through here (fp32, like the reference's Eigen
    GEMMs); experiments that model reduced-precision operands replace this one function."""
    return np.matmul(a, b)


def padded(count: int) -> int:
    """Arena slot size: each view is padded to 8 floats (opennn/tensor_utilities.cpp:472-487)."""
    return (count + 7) & ~7


# --------------------------------------------------------------------------------------
# Embedding
# --------------------------------------------------------------------------------------

def positional_encoding(sequence_length: int, embedding_dimension: int) -> np.ndarray:
    """opennn/embedding_layer.cpp:74-85: first half sin, second half cos (not interleaved);
    the exponent j/half_depth is a float division, pow/sin/cos run in double."""
    half_depth = F32(embedding_dimension) / F32(2)
    half = int(half_depth)
    table = np.zeros((sequence_length, embedding_dimension), dtype=F32)
    positions = np.arange(sequence_length, dtype=np.float64)[:, None]
    for j in range(embedding_dimension):
        if j < half:
            exponent = np.float64(F32(j) / half_depth)
            table[:, j] = np.sin(positions[:, 0] / np.power(10000.0, exponent)).astype(F32)
        else:
            exponent = np.float64(F32(j - half) / half_depth)
            table[:, j] = np.cos(positions[:, 0] / np.power(10000.0, exponent)).astype(F32)
    return table


def token_index(ids: np.ndarray) -> np.ndarray:
    """static_cast<Index>(float): truncation toward zero (opennn/embedding_layer.cpp:166)."""
    return np.trunc(ids).astype(np.int64)


def embedding_forward(ids, weights, pe, scale=True, add_pe=True):
    """opennn/embedding_layer.cpp:147-186.  ids [B,S] floats; weights [V,E]; pe [S,E]."""
    B, S = ids.shape
    V, E = weights.shape
    idx = token_index(ids)
    valid = (idx >= 0) & (idx < V)
    out = np.zeros((B, S, E), dtype=F32)
    out[valid] = weights[idx[valid]]
    if scale:
        out = out * np.sqrt(F32(E))
    if add_pe:
        positive = idx > 0
        out = out + np.where(positive[:, :, None], pe[None, :S, :], F32(0))
    return out.astype(F32)


def embedding_backward(ids, d_out, vocabulary_size, scale=True):
    """opennn/embedding_layer.cpp:193-226: scatter-add of sqrt(E)*dY, row 0 forced to zero."""
    B, S, E = d_out.shape
    idx = token_index(ids).reshape(-1)
    g = d_out.reshape(B * S, E).astype(F32)
    if scale:
        g = g * np.sqrt(F32(E))
    d_weights = np.zeros((vocabulary_size, E), dtype=F32)
    valid = (idx >= 0) & (idx < vocabulary_size)
    np.add.at(d_weights, idx[valid], g[valid])
    d_weights[0] = 0
    return d_weights


# --------------------------------------------------------------------------------------
# Normalization3d
# --------------------------------------------------------------------------------------

def layernorm_forward(x, gammas, betas):
    """opennn/normalization_layer_3d.cpp:87-125.  Returns y, mean, std, x_hat;
    std = sqrt(biased variance + EPSILON)."""
    mean = x.mean(axis=-1, dtype=F32, keepdims=True)
    centered = x - mean
    variance = np.mean(centered * centered, axis=-1, dtype=F32, keepdims=True)
    std = np.sqrt(variance + EPSILON).astype(F32)
    x_hat = (centered / std).astype(F32)
    y = (x_hat * gammas + betas).astype(F32)
    return y, mean[..., 0], std[..., 0], x_hat


def layernorm_backward(d_y, x_hat, std, gammas):
    """opennn/normalization_layer_3d.cpp:128-188."""
    E = d_y.shape[-1]
    d_gamma = (d_y * x_hat).reshape(-1, E).sum(axis=0, dtype=F32)
    d_beta = d_y.reshape(-1, E).sum(axis=0, dtype=F32)
    D = (d_y * gammas).astype(F32)
    sum_D = D.sum(axis=-1, dtype=F32, keepdims=True)
    sum_D_xhat = (D * x_hat).sum(axis=-1, dtype=F32, keepdims=True)
    inv_E = F32(1.0) / F32(E)
    d_x = (D - sum_D * inv_E - x_hat * sum_D_xhat * inv_E) / std[..., None]
    return d_x.astype(F32), d_gamma, d_beta


# --------------------------------------------------------------------------------------
# Dense<3>
# --------------------------------------------------------------------------------------

def softmax_last(y):
    """opennn/layer.cpp:338-371 (3-D) and 326-335 (2-D): max-subtracted exp over the last dim."""
    m = y.max(axis=-1, keepdims=True)
    e = np.exp((y - m).astype(F32)).astype(F32)
    s = e.sum(axis=-1, dtype=F32, keepdims=True)
    return (e * (F32(1.0) / s)).astype(F32)


def dense_forward(x, weights, biases, activation):
    """opennn/dense_layer.h:767-813 -> layer.h:305-340 (X.W + b) -> layer.h:122-152.
    Returns (outputs, activation_derivatives)."""
    rows = x.reshape(-1, x.shape[-1])
    combos = (_mm(rows, weights) + biases).astype(F32).reshape(*x.shape[:-1], weights.shape[1])
    if activation == "Linear":
        return combos, np.ones_like(combos)
    if activation == "RectifiedLinear":
        return np.maximum(combos, F32(0)), (combos > 0).astype(F32)
    if activation == "Softmax":
        return softmax_last(combos), None
    if activation == "Sigmoid":
        # opennn/layer.h:196-204: y = 1 / (1 + exp(-x)), derivative y (1 - y)
        y = (F32(1) / (F32(1) + np.exp(-combos).astype(F32))).astype(F32)
        return y, (y * (F32(1) - y)).astype(F32)
    raise ValueError(activation)


def dense_backward(x, weights, d_y, activation_derivatives, activation):
    """opennn/dense_layer.h:816-866: delta = dY*act' (Softmax: delta = dY, the loss already
    delivers dlogits), dW = X^T delta, db = colsum(delta), dX = delta W^T."""
    rows = x.reshape(-1, x.shape[-1])
    delta = d_y.reshape(-1, d_y.shape[-1])
    if activation != "Softmax":
        delta = delta * activation_derivatives.reshape(delta.shape)
    d_w = _mm(rows.T, delta).astype(F32)
    d_b = delta.sum(axis=0, dtype=F32)
    d_x = _mm(delta, weights.T).astype(F32).reshape(x.shape)
    return d_x, d_w, d_b


# --------------------------------------------------------------------------------------
# Pooling3d (sequence pooling in front of a classification head)
# --------------------------------------------------------------------------------------

def pooling3d_forward(x, method):
    """opennn/pooling_layer_3d.cpp:77-148.  x [B,S,E] -> y [B,E].  MaxPooling: maximum over the sequence, the FIRST
    position winning ties (strict >, :101-108), its index kept for the backward pass.  AveragePooling: mean over the
    rows that are not padding, a padding row being one whose features are all exactly zero (:119-141); a sample of
    nothing but padding gives zeros."""
    if method == "MaxPooling":
        indices = np.argmax(x, axis=1)                                    # first occurrence of the maximum
        return np.take_along_axis(x, indices[:, None, :], axis=1)[:, 0, :].astype(F32), indices
    valid = np.any(x != 0, axis=2)                                        # [B,S]
    y = np.zeros((x.shape[0], x.shape[2]), dtype=F32)
    for b in range(x.shape[0]):
        for s in range(x.shape[1]):                                       # sequential float accumulation, as :134-135
            if valid[b, s]:
                y[b] += x[b, s]
        count = int(valid[b].sum())
        if count > 0:
            y[b] /= F32(count)
    return y, valid


def pooling3d_backward(x, d_y, method, saved):
    """opennn/pooling_layer_3d.cpp:151-232.  MaxPooling routes each output gradient to the stored position, zeros
    elsewhere; AveragePooling gives every non-padding row d_y / count and padding rows zero."""
    d_x = np.zeros_like(x, dtype=F32)
    if method == "MaxPooling":
        np.put_along_axis(d_x, saved[:, None, :], d_y[:, None, :].astype(F32), axis=1)
        return d_x
    for b in range(x.shape[0]):
        count = int(saved[b].sum())
        if count == 0:
            continue
        inverse = F32(1.0) / F32(count)
        d_x[b, saved[b]] = (d_y[b] * inverse).astype(F32)
    return d_x


# --------------------------------------------------------------------------------------
# MultiHeadAttention
# --------------------------------------------------------------------------------------

def _split_heads(t, H):
    B, S, E = t.shape
    return t.reshape(B, S, H, E // H).transpose(0, 2, 1, 3)  # [B,H,S,hd]


def _merge_heads(t):
    B, H, S, hd = t.shape
    return t.transpose(0, 2, 1, 3).reshape(B, S, H * hd)


def key_padding_flags(source):
    """opennn/multihead_attention_layer.cpp:574-603: a source row is padding when every
    feature has |x| <= 1e-7 (data-dependent, not token ids)."""
    return np.all(np.abs(source) <= F32(1e-7), axis=-1)  # [B,Sk]


def mha_forward(xq, xs, p, H, causal):
    """opennn/multihead_attention_layer.cpp:183-282.  p: dict Wq,bq,Wk,bk,Wv,bv,Wo,bo
    (weights [E,E] in x out; head h = columns h*hd..).  Returns y and the saved state."""
    B, Sq, E = xq.shape
    Sk = xs.shape[1]
    hd = E // H
    scaling = F32(1.0) / np.sqrt(F32(hd))
    q = _split_heads((_mm(xq.reshape(-1, E), p["Wq"]) + p["bq"]).astype(F32).reshape(B, Sq, E), H)
    k = _split_heads((_mm(xs.reshape(-1, E), p["Wk"]) + p["bk"]).astype(F32).reshape(B, Sk, E), H)
    v = _split_heads((_mm(xs.reshape(-1, E), p["Wv"]) + p["bv"]).astype(F32).reshape(B, Sk, E), H)
    scores = (_mm(q, k.transpose(0, 1, 3, 2)) * scaling).astype(F32)  # [B,H,Sq,Sk]
    pad = key_padding_flags(xs)
    scores = np.where(pad[:, None, None, :], F32(-1e9), scores)            # :600 overwrite
    if causal:
        future = np.arange(Sk)[None, :] > np.arange(Sq)[:, None]          # :157 column > row
        scores = np.where(future[None, None], F32(-np.inf), scores)        # :570 additive -inf
    weights = softmax_last(scores)
    concat = _merge_heads(_mm(weights, v).astype(F32))              # [B,Sq,E]
    y = (_mm(concat.reshape(-1, E), p["Wo"]) + p["bo"]).astype(F32).reshape(B, Sq, E)
    saved = dict(q=q, k=k, v=v, weights=weights, concat=concat)
    return y, saved


def mha_backward(xq, xs, p, H, saved, d_y, self_attention):
    """opennn/multihead_attention_layer.cpp:285-454 and 493-553.
    Returns gradients dict (same keys as p, prefixed d) and dXq, dXs (dXs None for self)."""
    B, Sq, E = xq.shape
    Sk = xs.shape[1]
    hd = E // H
    scaling = F32(1.0) / np.sqrt(F32(hd))
    q, k, v, w, concat = saved["q"], saved["k"], saved["v"], saved["weights"], saved["concat"]
    dy = d_y.reshape(-1, E)
    g = {}
    g["dWo"] = _mm(concat.reshape(-1, E).T, dy).astype(F32)
    g["dbo"] = dy.sum(axis=0, dtype=F32)
    d_concat = _mm(dy, p["Wo"].T).astype(F32).reshape(B, Sq, E)
    d_o = _split_heads(d_concat, H)                                       # [B,H,Sq,hd]
    d_v = _mm(w.transpose(0, 1, 3, 2), d_o).astype(F32)
    d_w = _mm(d_o, v.transpose(0, 1, 3, 2)).astype(F32)
    dot = (w * d_w).sum(axis=-1, dtype=F32, keepdims=True)
    d_s = (w * (d_w - dot)).astype(F32)
    d_q = (_mm(d_s, k) * scaling).astype(F32)
    d_k = (_mm(d_s.transpose(0, 1, 3, 2), q) * scaling).astype(F32)

    def projection_gradient(d_head, x, W):
        d = _merge_heads(d_head).reshape(-1, E)
        return _mm(d, W.T).astype(F32).reshape(x.shape), _mm(x.reshape(-1, E).T, d).astype(F32), d.sum(axis=0, dtype=F32)

    d_xq, g["dWq"], g["dbq"] = projection_gradient(d_q, xq, p["Wq"])
    d_xk, g["dWk"], g["dbk"] = projection_gradient(d_k, xs, p["Wk"])
    d_xv, g["dWv"], g["dbv"] = projection_gradient(d_v, xs, p["Wv"])
    if self_attention:
        return g, (d_xq + d_xk + d_xv).astype(F32), None
    return g, d_xq, (d_xk + d_xv).astype(F32)


# --------------------------------------------------------------------------------------
# CrossEntropyError2d (several classes)
# --------------------------------------------------------------------------------------

def ce2d_error(probabilities, targets):
    """opennn/cross_entropy_error.cpp:58-77: -sum(t * log(y + eps)) / samples, eps = FLT_EPSILON."""
    samples = probabilities.shape[0]
    terms = (targets * np.log(probabilities + EPSILON)).astype(F32)
    return F32(terms.sum(dtype=F32) / F32(-samples))


def ce2d_output_gradients(probabilities, targets):
    """opennn/cross_entropy_error.cpp:114-134: (y - t) / samples -- the softmax Jacobian is folded in, the Softmax
    Dense layer passes it on unchanged (dense_layer.h:834-840)."""
    return ((probabilities - targets) / F32(probabilities.shape[0])).astype(F32)


def ce2d_binary_error(outputs, targets):
    """opennn/cross_entropy_error.cpp:36-55 (one output): y clipped to [eps, 1 - eps];
    -sum(t log y + (1 - t) log(1 - y)) / samples; NaN or infinity becomes 10."""
    samples = outputs.shape[0]
    y = np.minimum(np.maximum(outputs, EPSILON), F32(1) - EPSILON).astype(F32)
    terms = (targets * np.log(y) + (F32(1) - targets) * np.log(F32(1) - y)).astype(F32)
    error = F32(terms.sum(dtype=F32) / F32(-samples))
    return error if np.isfinite(error) else F32(10)


def ce2d_binary_output_gradients(outputs, targets):
    """opennn/cross_entropy_error.cpp:90-110: (-t / (y + eps) + (1 - t) / (1 - y + eps)) / samples; the Sigmoid layer
    behind it multiplies by y (1 - y)."""
    samples = F32(outputs.shape[0])
    return ((-targets / (outputs + EPSILON) + (F32(1) - targets) / (F32(1) - outputs + EPSILON)) / samples).astype(F32)


# --------------------------------------------------------------------------------------
# CrossEntropyError3d
# --------------------------------------------------------------------------------------

def ce3d_error(probabilities, targets):
    """opennn/cross_entropy_error_3d.cpp:78-136.  Returns (error, accuracy, active_count).
    Active = 0 < int(target) < V; loss term = -log(p[target] + EPSILON)."""
    B, S, V = probabilities.shape
    t = token_index(targets)
    active = (t > 0) & (t < V)
    count = int(active.sum())
    if count == 0:
        return F32(0), F32(0), 0
    rows = probabilities[active]
    picked = rows[np.arange(count), t[active]]
    total = F32(-np.log((picked + EPSILON).astype(F32)).astype(F32).sum(dtype=F32))
    correct = int((rows.argmax(axis=-1) == t[active]).sum())
    return F32(total / F32(count)), F32(F32(correct) / F32(count)), count


def ce3d_output_gradients(probabilities, targets, active_count=None):
    """opennn/cross_entropy_error_3d.cpp:154-247: (p - onehot)/active on active tokens, 0 elsewhere.
    active_count overrides the divisor: a data-parallel rank scales its shard by the count of
    the WHOLE batch, so that the sum of the ranks' gradients is the gradient of the whole batch."""
    B, S, V = probabilities.shape
    t = token_index(targets)
    active = (t > 0) & (t < V)
    count = int(active.sum())
    divisor = count if active_count is None else int(active_count)
    scale = F32(1.0) / F32(divisor) if divisor > 0 else F32(0)
    grad = np.zeros_like(probabilities, dtype=F32)
    onehot = np.zeros((count, V), dtype=F32)
    onehot[np.arange(count), t[active]] = 1
    grad[active] = (probabilities[active] - onehot) * scale
    return grad


# --------------------------------------------------------------------------------------
# Adam
# --------------------------------------------------------------------------------------

def adam_update(parameters, gradient, m, v, iteration, lr=1e-3, beta_1=0.9, beta_2=0.999, clip_norm=1.0, norm=None):
    """opennn/adaptive_moment_estimation.cpp:444-473.  `iteration` is the value AFTER the
    increment (the loop starts at 1, so the first step passes 2).  Updates in place.
    `norm`: the gradient norm to clip by when `gradient` is only a part of the whole gradient (a
    data-parallel rank that updates its share of the arena clips by the norm of the whole)."""
    lr, beta_1, beta_2, clip_norm = F32(lr), F32(beta_1), F32(beta_2), F32(clip_norm)
    bc1 = F32(1) - F32(np.power(beta_1, F32(iteration)))
    bc2 = F32(1) - F32(np.power(beta_2, F32(iteration)))
    norm = F32(np.sqrt(np.sum(gradient.astype(np.float64) ** 2))) if norm is None else F32(norm)
    g = gradient
    if clip_norm > 0 and norm > clip_norm:
        g = (gradient * (clip_norm / norm)).astype(F32)
    m[:] = beta_1 * m + (F32(1) - beta_1) * g
    v[:] = beta_2 * v + (F32(1) - beta_2) * g * g
    parameters -= (lr * (m / bc1) / (np.sqrt(v / bc2) + EPSILON)).astype(F32)
    return norm


# --------------------------------------------------------------------------------------
# Network graph (NeuralNetwork + Transformer builder)
# --------------------------------------------------------------------------------------

PARAMETER_SHAPES = {
    # view order inside the arena:
    "Embedding": lambda l: [("weights", (l["V"], l["E"]))],                      # embedding_layer.cpp:60
    "MultiHeadAttention": lambda l: [("Wq", (l["E"], l["E"])), ("bq", (l["E"],)),  # multihead_attention_layer.cpp:105-108
                                     ("Wk", (l["E"], l["E"])), ("bk", (l["E"],)),
                                     ("Wv", (l["E"], l["E"])), ("bv", (l["E"],)),
                                     ("Wo", (l["E"], l["E"])), ("bo", (l["E"],))],
    "Addition3d": lambda l: [],
    "Normalization3d": lambda l: [("gammas", (l["E"],)), ("betas", (l["E"],))],  # normalization_layer_3d.cpp:49
    "Dense3d": lambda l: [("biases", (l["out"],)), ("weights", (l["in"], l["out"]))],  # dense_layer.h:484
    "Dense2d": lambda l: [("biases", (l["out"],)), ("weights", (l["in"], l["out"]))],  # the same template, rank 2
    "Pooling3d": lambda l: [],
}


class Network:
    """Layer DAG with one parameter arena and one gradient arena in the same layout
    (opennn/neural_network.cpp:66-94, 1489-1497).  Negative input index = external input:
    -1 decoder ids, -2 encoder ids (opennn/standard_networks.cpp:669-704)."""

    def __init__(self):
        self.layers = []

    def add(self, kind, inputs=None, **cfg):
        if inputs is None:
            inputs = [len(self.layers) - 1]
        self.layers.append(dict(kind=kind, inputs=list(inputs), **cfg))
        return len(self.layers) - 1

    def compile(self):
        offset = 0
        for layer in self.layers:
            layer["views"] = {}
            for name, shape in PARAMETER_SHAPES[layer["kind"]](layer):
                count = int(np.prod(shape))
                layer["views"][name] = (offset, shape)
                offset += padded(count)
            if layer["kind"] == "Embedding":
                layer["pe"] = positional_encoding(layer["S"], layer["E"])
        self.parameters_size = offset
        self.consumers = [[] for _ in self.layers]
        for i, layer in enumerate(self.layers):
            for port, src in enumerate(layer["inputs"]):
                if src >= 0:
                    self.consumers[src].append((i, port))
        return self

    def views(self, arena, layer):
        return {name: arena[o:o + int(np.prod(shape))].reshape(shape) for name, (o, shape) in layer["views"].items()}

    def default_parameters(self, rng):
        """The reference's own initial distributions (dense_layer.h:581-597, embedding_layer.cpp:114-126,
        normalization_layer_3d.cpp:72-79, MHA U(-0.1,0.1)); drawn from OUR seeded generator."""
        arena = np.zeros(self.parameters_size, dtype=F32)
        for layer in self.layers:
            v = self.views(arena, layer)
            kind = layer["kind"]
            if kind == "Embedding":
                v["weights"][:] = F32(0.05) * rng.uniform(-1, 1, v["weights"].shape).astype(F32)
                v["weights"][0] = 0
            elif kind == "MultiHeadAttention":
                for name in v:
                    v[name][:] = rng.uniform(-0.1, 0.1, v[name].shape).astype(F32)
            elif kind == "Normalization3d":
                v["gammas"][:] = 1
            elif kind in ("Dense3d", "Dense2d"):
                v["weights"][:] = rng.uniform(-0.1, 0.1, v["weights"].shape).astype(F32)
        return arena

    def forward(self, arena, external):
        """opennn/neural_network.cpp:645-699.  external: {-1: decoder ids, -2: encoder ids}."""
        self.outputs = [None] * len(self.layers)
        self.saved = [None] * len(self.layers)
        for i, layer in enumerate(self.layers):
            ins = [external[s] if s < 0 else self.outputs[s] for s in layer["inputs"]]
            p = self.views(arena, layer)
            kind = layer["kind"]
            if kind == "Embedding":
                self.outputs[i] = embedding_forward(ins[0], p["weights"], layer["pe"])
            elif kind == "MultiHeadAttention":
                xs = ins[1] if len(ins) > 1 else ins[0]
                self.outputs[i], self.saved[i] = mha_forward(ins[0], xs, p, layer["H"], layer["causal"])
            elif kind == "Addition3d":
                self.outputs[i] = (ins[0] + ins[1]).astype(F32)       # addition_layer.h:65-76
            elif kind == "Normalization3d":
                y, mean, std, x_hat = layernorm_forward(ins[0], p["gammas"], p["betas"])
                self.outputs[i], self.saved[i] = y, (std, x_hat)
            elif kind in ("Dense3d", "Dense2d"):
                self.outputs[i], self.saved[i] = dense_forward(ins[0], p["weights"], p["biases"], layer["activation"])
            elif kind == "Pooling3d":
                self.outputs[i], self.saved[i] = pooling3d_forward(ins[0], layer["method"])
            self.layers[i]["_ins"] = ins
        return self.outputs[-1]

    def backward(self, arena, d_outputs):
        """opennn/loss.cpp:284-303: reverse layer walk; fan-out gradients are summed in
        consumer order (layer.cpp:285-291).  Returns the gradient arena."""
        gradient = np.zeros(self.parameters_size, dtype=F32)
        input_grads = [dict() for _ in self.layers]
        for i in range(len(self.layers) - 1, -1, -1):
            layer = self.layers[i]
            if i == len(self.layers) - 1:
                d_y = d_outputs
            else:
                parts = [input_grads[c][port] for c, port in self.consumers[i]]
                d_y = parts[0]
                for extra in parts[1:]:
                    d_y = (d_y + extra).astype(F32)
            ins = layer["_ins"]
            p = self.views(arena, layer)
            g = self.views(gradient, layer)
            kind = layer["kind"]
            if kind == "Embedding":
                g["weights"][:] = embedding_backward(ins[0], d_y, layer["V"])
            elif kind == "MultiHeadAttention":
                self_attention = len(ins) == 1
                xs = ins[0] if self_attention else ins[1]
                grads, d_xq, d_xs = mha_backward(ins[0], xs, p, layer["H"], self.saved[i], d_y, self_attention)
                for name in ("Wq", "bq", "Wk", "bk", "Wv", "bv", "Wo", "bo"):
                    g[name][:] = grads["d" + name]
                input_grads[i][0] = d_xq
                if not self_attention:
                    input_grads[i][1] = d_xs
            elif kind == "Addition3d":
                input_grads[i][0] = d_y                               # addition_layer.h:79-90
                input_grads[i][1] = d_y
            elif kind == "Normalization3d":
                std, x_hat = self.saved[i]
                d_x, g["gammas"][:], g["betas"][:] = layernorm_backward(d_y, x_hat, std, p["gammas"])
                input_grads[i][0] = d_x
            elif kind in ("Dense3d", "Dense2d"):
                d_x, g["weights"][:], g["biases"][:] = dense_backward(ins[0], p["weights"], d_y, self.saved[i], layer["activation"])
                input_grads[i][0] = d_x
            elif kind == "Pooling3d":
                input_grads[i][0] = pooling3d_backward(ins[0], d_y, layer["method"], self.saved[i])
        return gradient

    def train_step_2d(self, arena, m, v, iteration, ids, targets, lr=1e-3):
        """The same loop body with CrossEntropyError2d on a classifier: targets are one-hot rows [B, classes]."""
        probabilities = self.forward(arena, {-1: ids})
        if probabilities.shape[-1] == 1:                     # one output: the binary form of the loss
            error = ce2d_binary_error(probabilities, targets)
            gradient = self.backward(arena, ce2d_binary_output_gradients(probabilities, targets))
        else:
            error = ce2d_error(probabilities, targets)
            gradient = self.backward(arena, ce2d_output_gradients(probabilities, targets))
        iteration += 1
        adam_update(arena, gradient, m, v, iteration, lr=lr)
        return error, gradient, iteration

    def train_step(self, arena, m, v, iteration, external, targets, lr=1e-3):
        """Loop body of opennn/adaptive_moment_estimation.cpp:249-284 (regularisation "None").
        Returns (error, accuracy, gradient, iteration_after)."""
        probabilities = self.forward(arena, external)
        error, accuracy, _ = ce3d_error(probabilities, targets)
        gradient = self.backward(arena, ce3d_output_gradients(probabilities, targets))
        iteration += 1
        adam_update(arena, gradient, m, v, iteration, lr=lr)
        return error, accuracy, gradient, iteration


def _encoder_block(net, S, E, H, F, source):
    attention = net.add("MultiHeadAttention", [source], Sq=S, Sk=S, E=E, H=H, causal=False)
    net.add("Addition3d", [source, attention], E=E)
    norm_1 = net.add("Normalization3d", S=S, E=E)
    net.add("Dense3d", **{"in": E, "out": F, "activation": "RectifiedLinear"})
    dense = net.add("Dense3d", **{"in": F, "out": E, "activation": "Linear"})
    net.add("Addition3d", [norm_1, dense], E=E)
    return net.add("Normalization3d", S=S, E=E)


def build_text_classifier(V, S, E, H, hidden, classes):
    """opennn/standard_networks.cpp:575-615: Embedding (scaled, with positions) -> self-attention -> max pooling over
    the sequence -> Dense<2> ReLU layers -> Dense<2> Softmax, or Sigmoid for a single output."""
    net = Network()
    net.add("Embedding", [-1], V=V, S=S, E=E)
    net.add("MultiHeadAttention", Sq=S, Sk=S, E=E, H=H, causal=False)
    net.add("Pooling3d", method="MaxPooling")
    width = E
    for size in hidden:
        net.add("Dense2d", **{"in": width, "out": size, "activation": "RectifiedLinear"})
        width = size
    net.add("Dense2d", **{"in": width, "out": classes, "activation": "Softmax" if classes > 1 else "Sigmoid"})
    return net.compile()


def greedy_decode(net, arena, source_ids, S_dec, start=2, end=3):
    """The decoding loop of opennn/standard_networks.cpp:1002-1035 on token ids (the tokeniser and the vocabulary
    maps around it are not part of this path): the target starts as [START, PAD, ...]; step i runs the whole network
    on it (inference: the last layer gives probabilities), takes the arg-max of the distribution at position i - 1
    (first index on ties, opennn/tensor_utilities.cpp maximal_index) as token i and stops after END.  source_ids
    [B, S_in]; every row is decoded independently.  Returns ids [B, S_dec] (PAD after END)."""
    B = source_ids.shape[0]
    target = np.zeros((B, S_dec), dtype=F32)
    target[:, 0] = start
    finished = np.zeros(B, dtype=bool)
    for i in range(1, S_dec):
        probabilities = net.forward(arena, {-1: target, -2: source_ids})
        best = np.argmax(probabilities[:, i - 1, :], axis=-1)
        for b in range(B):
            if finished[b]:
                continue
            target[b, i] = best[b]
            if best[b] == end:
                finished[b] = True
        if finished.all():
            break
    return target


def build_transformer(S_in, S_dec, V_in, V_out, E, H, F, L):
    """opennn/standard_networks.cpp:638-907: post-norm encoder-decoder, 2 + 7L + 10L + 1 layers."""
    net = Network()
    decoder = net.add("Embedding", [-1], V=V_out, S=S_dec, E=E)
    encoder = net.add("Embedding", [-2], V=V_in, S=S_in, E=E)
    for _ in range(L):
        encoder = _encoder_block(net, S_in, E, H, F, encoder)
    for _ in range(L):
        attention = net.add("MultiHeadAttention", [decoder], Sq=S_dec, Sk=S_dec, E=E, H=H, causal=True)
        net.add("Addition3d", [decoder, attention], E=E)
        norm_1 = net.add("Normalization3d", S=S_dec, E=E)
        cross = net.add("MultiHeadAttention", [norm_1, encoder], Sq=S_dec, Sk=S_in, E=E, H=H, causal=False)
        net.add("Addition3d", [norm_1, cross], E=E)
        norm_2 = net.add("Normalization3d", S=S_dec, E=E)
        net.add("Dense3d", **{"in": E, "out": F, "activation": "RectifiedLinear"})
        dense = net.add("Dense3d", **{"in": F, "out": E, "activation": "Linear"})
        net.add("Addition3d", [norm_2, dense], E=E)
        decoder = net.add("Normalization3d", S=S_dec, E=E)
    net.add("Dense3d", **{"in": E, "out": V_out, "activation": "Softmax"})
    return net.compile()


def build_decoder_only(S, V, E, H, F, L):
    """Decoder-only stack assembled the way Transformer::set assembles its decoder minus
    cross-attention (causal self-attention -> add -> norm -> FFN -> add -> norm)."""
    net = Network()
    current = net.add("Embedding", [-1], V=V, S=S, E=E)
    for _ in range(L):
        attention = net.add("MultiHeadAttention", [current], Sq=S, Sk=S, E=E, H=H, causal=True)
        net.add("Addition3d", [current, attention], E=E)
        norm_1 = net.add("Normalization3d", S=S, E=E)
        net.add("Dense3d", **{"in": E, "out": F, "activation": "RectifiedLinear"})
        dense = net.add("Dense3d", **{"in": F, "out": E, "activation": "Linear"})
        net.add("Addition3d", [norm_1, dense], E=E)
        current = net.add("Normalization3d", S=S, E=E)
    net.add("Dense3d", **{"in": E, "out": V, "activation": "Softmax"})
    return net.compile()


# --------------------------------------------------------------------------------------
# Seeded synthetic inputs shared by the oracle, the reference harness and the CUDA path
# --------------------------------------------------------------------------------------

def synthetic_ids(rng, batch, sequence_length, vocabulary, min_length, max_length):
    """Token ids uniform in [1, vocabulary), per-row length ~U[min_length, max_length],
    right-padded with id 0; stored as floats holding integers (dataset.h:525-558)."""
    ids = rng.integers(1, vocabulary, size=(batch, sequence_length)).astype(F32)
    lengths = rng.integers(min_length, max_length + 1, size=batch)
    ids[np.arange(sequence_length)[None, :] >= lengths[:, None]] = 0
    return ids
