"""ctypes binding of libonn_b200.so (include/onn_b200.h).

PyTorch is used here only to own device memory and streams: every function below passes
raw device pointers and sizes across the C ABI.  There is no fallback: if the library is
missing, import fails; if a call returns a non-zero status, OnnError is raised.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libonn_b200.so")

OK = 0
ACCUMULATE = 2
DEFER_SOFTMAX = 8
DELTA_READY = 16
ACT_LINEAR, ACT_RELU, ACT_SOFTMAX = 0, 1, 2
ACTIVATIONS = {"Linear": ACT_LINEAR, "RectifiedLinear": ACT_RELU, "Softmax": ACT_SOFTMAX, "Sigmoid": 3, "Logistic": 3}


class OnnError(RuntimeError):
    pass


class GemmArgs(C.Structure):
    _fields_ = [("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p),
                ("bias", C.c_void_p), ("relu_mask", C.c_void_p),
                ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
                ("a_major", C.c_int32), ("b_major", C.c_int32),
                ("batch_inner", C.c_int32), ("batch_outer", C.c_int32),
                ("a_stride_inner", C.c_int64), ("a_stride_outer", C.c_int64),
                ("b_stride_inner", C.c_int64), ("b_stride_outer", C.c_int64),
                ("c_stride_inner", C.c_int64), ("c_stride_outer", C.c_int64),
                ("alpha", C.c_float), ("relu", C.c_int32), ("split_k", C.c_int32), ("flags", C.c_uint32),
                ("colsum_out", C.c_void_p), ("colsum_stride_inner", C.c_int64),
                ("relu_bits_out", C.c_void_p), ("relu_bits", C.c_void_p), ("relu_bits_ld", C.c_int64),
                ("k_parts", C.c_int32), ("a_stride_part", C.c_int64), ("b_stride_part", C.c_int64)]


class MhaParams(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("Wq", "bq", "Wk", "bk", "Wv", "bv", "Wo", "bo")]


class MhaGrads(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("dWq", "dbq", "dWk", "dbk", "dWv", "dbv", "dWo", "dbo")]


EXPORTS = [
    "onn_status_string", "onn_version", "onn_gemm", "onn_gemm_set_mode", "onn_mha_set_kv_grad_by_recomputation", "onn_gemm_device_status",
    "onn_launch_count", "onn_launch_count_add", "onn_selftest_bounded_wait", "onn_embedding_fwd", "onn_embedding_bwd", "onn_ids_to_float",
    "onn_layernorm_fwd", "onn_layernorm_bwd_workspace_floats", "onn_layernorm_bwd", "onn_layernorm_bwd_static", "onn_add",
    "onn_relu_bits_words_per_row", "onn_dense_fwd", "onn_dense_bwd", "onn_pooling3d_fwd", "onn_pooling3d_bwd", "onn_softmax_rows",
    "onn_mha_fwd_workspace_floats", "onn_mha_bwd_workspace_floats", "onn_mha_fwd", "onn_mha_bwd",
    "onn_mha_attention_weights", "onn_ce2d_fwd_bwd", "onn_ce2d_binary_fwd_bwd", "onn_dense_fwd_shared_input", "onn_greedy_next_token", "onn_greedy_next_token_rows", "onn_greedy_next_token_logits", "onn_decode_attention", "onn_rows_are_zero", "onn_ce3d_count_active", "onn_ce3d_fwd_bwd",
    "onn_grad_sqnorm_workspace_floats", "onn_grad_sqnorm", "onn_adam", "onn_adam_guarded", "onn_device_status_gather", "onn_set_sm_limit", "onn_set_dynamic_work", "onn_selftest_hold_sms",
    "onn_dp_unique_id", "onn_dp_init", "onn_dp_init_config", "onn_dp_world", "onn_dp_rank", "onn_dp_allreduce", "onn_dp_reduce_scatter",
    "onn_dp_all_gather", "onn_dp_zero", "onn_dp_wait", "onn_dp_mark", "onn_dp_wait_mark", "onn_dp_mark_failed", "onn_dp_finalize",
]

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OnnError(f"{LIB_PATH} is missing: run `python -m opennn_b200._build` (there is no fallback path)")
        L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        L.onn_status_string.restype = C.c_char_p
        L.onn_launch_count.restype = C.c_uint64
        L.onn_relu_bits_words_per_row.restype = C.c_int64
        for name in ("onn_layernorm_bwd_workspace_floats",
                     "onn_mha_fwd_workspace_floats", "onn_mha_bwd_workspace_floats",
                     "onn_grad_sqnorm_workspace_floats"):
            getattr(L, name).restype = C.c_size_t
            getattr(L, name).argtypes = None
        L.onn_mha_attention_weights.restype = C.c_void_p
        _lib = L
    return _lib


def check(status: int, what: str = "onn call"):
    if status != OK:
        raise OnnError(f"{what} failed: {lib().onn_status_string(status).decode()} ({status})")


def ptr(t):
    if t is None:
        return C.c_void_p(0)
    assert t.is_cuda and t.is_contiguous(), "device, contiguous tensors only"
    return C.c_void_p(t.data_ptr())


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def i64(x):
    return C.c_int64(int(x))


def f32(x):
    return C.c_float(float(x))


def _empty(n, dtype=torch.float32):
    return torch.empty(max(int(n), 1), dtype=dtype, device="cuda")


# ----------------------------------------------------------------------------------------
# thin wrappers (allocate outputs / workspace with torch, call the C ABI)
# ----------------------------------------------------------------------------------------

def gemm(A, B, Cmat, M, N, K, lda, ldb, ldc, a_major=0, b_major=1, bias=None, relu_mask=None, alpha=1.0,
         relu=False, split_k=0, flags=0, batch_inner=1, batch_outer=1, a_strides=(0, 0), b_strides=(0, 0), c_strides=(0, 0),
         colsum_out=None, colsum_stride_inner=0, relu_bits_out=None, relu_bits=None, relu_bits_ld=0,
         k_parts=0, part_strides=(0, 0)):
    g = GemmArgs()
    g.A, g.B, g.C = A.data_ptr(), B.data_ptr(), Cmat.data_ptr()
    g.bias = bias.data_ptr() if bias is not None else None
    g.relu_mask = relu_mask.data_ptr() if relu_mask is not None else None
    g.M, g.N, g.K, g.lda, g.ldb, g.ldc = M, N, K, lda, ldb, ldc
    g.a_major, g.b_major = a_major, b_major
    g.batch_inner, g.batch_outer = batch_inner, batch_outer
    g.a_stride_inner, g.a_stride_outer = a_strides
    g.b_stride_inner, g.b_stride_outer = b_strides
    g.c_stride_inner, g.c_stride_outer = c_strides
    g.alpha, g.relu, g.split_k, g.flags = alpha, int(relu), split_k, flags
    g.colsum_out = colsum_out.data_ptr() if colsum_out is not None else None
    g.colsum_stride_inner = colsum_stride_inner
    g.relu_bits_out = relu_bits_out.data_ptr() if relu_bits_out is not None else None
    g.relu_bits = relu_bits.data_ptr() if relu_bits is not None else None
    g.relu_bits_ld = relu_bits_ld
    g.k_parts = k_parts
    g.a_stride_part, g.b_stride_part = part_strides
    check(lib().onn_gemm(C.byref(g), stream_ptr()), "onn_gemm")


def embedding_fwd(ids, W, PE, scale=True, add_pe=True, flags=0, want_flags=False):
    B, S = ids.shape
    V, E = W.shape
    out = torch.empty(B, S, E, device="cuda")
    zero = torch.empty(B * S, dtype=torch.uint8, device="cuda") if want_flags else None
    check(lib().onn_embedding_fwd(ptr(ids), ptr(W), ptr(PE), ptr(out), ptr(zero), i64(B), i64(S), i64(E), i64(V),
                                  int(scale), int(add_pe), C.c_uint32(flags), stream_ptr()), "onn_embedding_fwd")
    return (out, zero) if want_flags else out


def embedding_bwd(ids, dY, V, scale=True, dY2=None):
    B, S, E = dY.shape
    dW = torch.zeros(V, E, device="cuda")
    check(lib().onn_embedding_bwd(ptr(ids), ptr(dY), ptr(dY2), ptr(dW), i64(B), i64(S), i64(E), i64(V), int(scale),
                                  stream_ptr()), "onn_embedding_bwd")
    return dW


def layernorm_fwd(A, gamma, beta, R=None, eps=None, flags=0, want_sum=False):
    E = A.shape[-1]
    rows = A.numel() // E
    eps = torch.finfo(torch.float32).eps if eps is None else eps
    Y = torch.empty_like(A)
    total = torch.empty_like(A) if want_sum else None
    mean = torch.empty(rows, device="cuda")
    inv_std = torch.empty(rows, device="cuda")
    check(lib().onn_layernorm_fwd(ptr(A), ptr(R), ptr(gamma), ptr(beta), ptr(Y), ptr(total), ptr(mean), ptr(inv_std),
                                  C.c_void_p(0), i64(rows), i64(E), f32(eps), C.c_uint32(flags), stream_ptr()), "onn_layernorm_fwd")
    return Y, mean, inv_std, total


def layernorm_bwd(dY, X, mean, inv_std, gamma, dY2=None, dY3=None, flags=0, dx_colsum=None):
    E = X.shape[-1]
    rows = X.numel() // E
    dX = torch.empty_like(X)
    dgamma = torch.zeros(E, device="cuda")
    dbeta = torch.zeros(E, device="cuda")
    ws = _empty(lib().onn_layernorm_bwd_workspace_floats(i64(rows), i64(E)))
    check(lib().onn_layernorm_bwd(ptr(dY), ptr(dY2), ptr(dY3), ptr(X), ptr(mean), ptr(inv_std), ptr(gamma), ptr(dX),
                                  ptr(dgamma), ptr(dbeta), ptr(dx_colsum), i64(rows), i64(E), ptr(ws), C.c_uint32(flags), stream_ptr()),
          "onn_layernorm_bwd")
    return dX, dgamma, dbeta


def add(a, b, flags=0):
    out = torch.empty_like(a)
    check(lib().onn_add(ptr(a), ptr(b), ptr(out), i64(a.numel()), C.c_uint32(flags), stream_ptr()), "onn_add")
    return out


def relu_bits_words_per_row(features):
    return (features + 31) // 32


def dense_fwd(X, W, b, activation, flags=0, want_relu_bits=False):
    in_f, out_f = W.shape
    rows = X.numel() // in_f
    Y = torch.empty(*X.shape[:-1], out_f, device="cuda")
    bits = torch.empty(rows, relu_bits_words_per_row(out_f), dtype=torch.int32, device="cuda") if want_relu_bits else None
    check(lib().onn_dense_fwd(ptr(X), ptr(W), ptr(b), ptr(Y), ptr(bits), i64(rows), i64(in_f), i64(out_f), ACTIVATIONS[activation],
                              C.c_uint32(flags), stream_ptr()), "onn_dense_fwd")
    return (Y, bits) if want_relu_bits else Y


def dense_bwd(X, W, Y, dY, activation, flags=0, need_dx=True, relu_mask=None, dx_colsum=None, relu_bits=None):
    in_f, out_f = W.shape
    rows = X.numel() // in_f
    dY = dY.clone()
    dW = torch.zeros_like(W)
    db = torch.zeros(out_f, device="cuda")
    dX = torch.empty_like(X) if need_dx else None
    check(lib().onn_dense_bwd(ptr(X), ptr(W), ptr(Y), ptr(dY), ptr(dW), ptr(db), ptr(dX), ptr(relu_mask), ptr(relu_bits), ptr(dx_colsum), i64(rows),
                              i64(in_f), i64(out_f), ACTIVATIONS[activation], C.c_uint32(flags), stream_ptr()), "onn_dense_bwd")
    return dX, dW, db


POOLING_METHODS = {"MaxPooling": 0, "AveragePooling": 1}


def pooling3d_fwd(x, method):
    B, S, E = x.shape
    y = torch.empty(B, E, device="cuda")
    argmax = torch.empty(B, E, dtype=torch.int32, device="cuda")
    valid = torch.empty(B * S, dtype=torch.uint8, device="cuda")
    count = torch.empty(B, dtype=torch.int32, device="cuda")
    check(lib().onn_pooling3d_fwd(ptr(x), ptr(y), ptr(argmax), ptr(valid), ptr(count), i64(B), i64(S), i64(E),
                                  POOLING_METHODS[method], stream_ptr()), "onn_pooling3d_fwd")
    return y, (argmax, valid, count)


def pooling3d_bwd(dy, saved, S, method):
    B, E = dy.shape
    argmax, valid, count = saved
    dx = torch.empty(B, S, E, device="cuda")
    check(lib().onn_pooling3d_bwd(ptr(dy), ptr(argmax), ptr(valid), ptr(count), ptr(dx), i64(B), i64(S), i64(E),
                                  POOLING_METHODS[method], stream_ptr()), "onn_pooling3d_bwd")
    return dx


def softmax_rows(Y):
    cols = Y.shape[-1]
    check(lib().onn_softmax_rows(ptr(Y), i64(Y.numel() // cols), i64(cols), stream_ptr()), "onn_softmax_rows")
    return Y


def _mha_params(p):
    s = MhaParams()
    for name in ("Wq", "bq", "Wk", "bk", "Wv", "bv", "Wo", "bo"):
        setattr(s, name, p[name].data_ptr())
    return s


def mha_fwd(Xq, Xs, p, H, causal, flags=0):
    B, Sq, E = Xq.shape
    Sk = Xs.shape[1]
    Y = torch.empty_like(Xq)
    ws = _empty(lib().onn_mha_fwd_workspace_floats(i64(B), i64(Sq), i64(Sk), i64(E), i64(H)))
    params = _mha_params(p)
    xs_ptr = ptr(Xq) if Xs is Xq else ptr(Xs)
    check(lib().onn_mha_fwd(ptr(Xq), xs_ptr, C.byref(params), C.c_void_p(0), ptr(Y), i64(B), i64(Sq), i64(Sk), i64(E), i64(H),
                            int(causal), ptr(ws), C.c_uint32(flags), stream_ptr()), "onn_mha_fwd")
    return Y, ws


def mha_attention_weights(ws, B, Sq, Sk, E, H):
    base = lib().onn_mha_attention_weights(ptr(ws), i64(B), i64(Sq), i64(Sk), i64(E), i64(H))
    offset = (base - ws.data_ptr()) // 4
    return ws[offset:offset + B * H * Sq * Sk].view(B, H, Sq, Sk)


def mha_bwd(Xq, Xs, p, H, causal, fwd_ws, dY, flags=0):
    B, Sq, E = Xq.shape
    Sk = Xs.shape[1]
    self_attention = Xs is Xq
    grads = {("d" + n): torch.zeros_like(p[n]) for n in ("Wq", "bq", "Wk", "bk", "Wv", "bv", "Wo", "bo")}
    g = MhaGrads()
    for name, t in grads.items():
        setattr(g, name, t.data_ptr())
    dXq = torch.empty_like(Xq)
    dXs = None if self_attention else torch.empty_like(Xs)
    ws = _empty(lib().onn_mha_bwd_workspace_floats(i64(B), i64(Sq), i64(Sk), i64(E), i64(H)))
    params = _mha_params(p)
    xs_ptr = ptr(Xq) if self_attention else ptr(Xs)
    check(lib().onn_mha_bwd(ptr(Xq), xs_ptr, C.byref(params), ptr(fwd_ws), ptr(dY), C.byref(g), ptr(dXq), ptr(dXs),
                            i64(B), i64(Sq), i64(Sk), i64(E), i64(H), int(causal), ptr(ws), C.c_uint32(flags), stream_ptr()),
          "onn_mha_bwd")
    return grads, dXq, dXs


def ce3d(logits, targets, inputs_are_probabilities=False, want_probabilities=False, flags=0):
    """Returns (error, accuracy, gradient, probabilities or None).  `logits` is consumed (overwritten)."""
    V = logits.shape[-1]
    rows = logits.numel() // V
    count = torch.empty(1, device="cuda")
    stats = torch.empty(4, device="cuda")
    scratch = torch.empty(2 * rows, device="cuda")
    probabilities = torch.empty_like(logits) if want_probabilities else None
    check(lib().onn_ce3d_count_active(ptr(targets), i64(rows), i64(V), ptr(count), stream_ptr()), "onn_ce3d_count_active")
    check(lib().onn_ce3d_fwd_bwd(ptr(logits), ptr(targets), ptr(count), ptr(probabilities), ptr(stats), ptr(scratch),
                                 i64(rows), i64(V), int(inputs_are_probabilities), C.c_uint32(flags), stream_ptr()), "onn_ce3d_fwd_bwd")
    loss_sum, correct, active, _ = stats.tolist()
    error = loss_sum / active if active > 0 else 0.0
    accuracy = correct / active if active > 0 else 0.0
    return error, accuracy, logits, probabilities


def ce2d(probabilities, targets):
    """CrossEntropyError2d with several classes.  Returns (error, gradient); `probabilities` is consumed (overwritten)."""
    classes = probabilities.shape[-1]
    rows = probabilities.numel() // classes
    stats = torch.empty(2, device="cuda")
    scratch = torch.empty(rows, device="cuda")
    check(lib().onn_ce2d_fwd_bwd(ptr(probabilities), ptr(targets), ptr(stats), ptr(scratch), i64(rows), i64(classes), stream_ptr()),
          "onn_ce2d_fwd_bwd")
    return float(stats[0]), probabilities


def ce2d_binary(outputs, targets, fold_sigmoid=False):
    """CrossEntropyError2d with one output per sample.  Returns (error, gradient or Sigmoid delta); `outputs` is consumed."""
    rows = outputs.numel()
    stats = torch.empty(2, device="cuda")
    scratch = torch.empty(rows, device="cuda")
    check(lib().onn_ce2d_binary_fwd_bwd(ptr(outputs), ptr(targets), ptr(stats), ptr(scratch), i64(rows), int(fold_sigmoid), stream_ptr()),
          "onn_ce2d_binary_fwd_bwd")
    return float(stats[0]), outputs


def dense_fwd_shared_input(x, weights, biases, outputs, pitches):
    """outputs[i][:, :out] = x @ weights[i] + biases[i]; outputs are preallocated, row pitch pitches[i] floats."""
    count = len(weights)
    rows, features = x.shape
    out = weights[0].shape[1]
    W = (C.c_void_p * count)(*[w.data_ptr() for w in weights])
    b = (C.c_void_p * count)(*[v.data_ptr() for v in biases]) if biases is not None else None
    Y = (C.c_void_p * count)(*[y.data_ptr() for y in outputs])
    ld = (C.c_int64 * count)(*pitches)
    check(lib().onn_dense_fwd_shared_input(ptr(x), W, b, Y, ld, count, i64(rows), i64(features), i64(out), stream_ptr()),
          "onn_dense_fwd_shared_input")


def decode_attention(q, k_cache, v_cache, key_is_pad, length, H, position_major=False):
    """One query row per sample against the first `length` cached keys and values.  q [B, E]; caches [B, S_cache, E];
    key_is_pad uint8 [B, S_cache] (or [S_cache, B] with position_major) or None.  Returns the context [B, E]."""
    B, S_cache, E = k_cache.shape
    out = torch.empty(B, E, device="cuda")
    strides = (1, B) if position_major else (S_cache, 1)
    check(lib().onn_decode_attention(ptr(q), ptr(k_cache), ptr(v_cache), ptr(key_is_pad), i64(strides[0]), i64(strides[1]), ptr(out),
                                     i64(B), i64(S_cache), i64(length), i64(E), i64(H), stream_ptr()), "onn_decode_attention")
    return out


def greedy_next_token_rows(probabilities, ids, finished, write_position, end_id):
    """probabilities [B, V]; ids float [B, S] (column write_position receives the arg-max of unfinished rows); finished int32 [B]."""
    B, V = probabilities.shape
    check(lib().onn_greedy_next_token_rows(ptr(probabilities), ptr(ids), ptr(finished), i64(B), i64(ids.shape[1]), i64(V),
                                           i64(write_position), int(end_id), stream_ptr()), "onn_greedy_next_token_rows")


def greedy_next_token_logits(logits, ids, finished, write_position, end_id):
    """As greedy_next_token_rows, from logits [B, V]: softmax and arg-max fused."""
    B, V = logits.shape
    check(lib().onn_greedy_next_token_logits(ptr(logits), ptr(ids), ptr(finished), i64(B), i64(ids.shape[1]), i64(V),
                                             i64(write_position), int(end_id), stream_ptr()), "onn_greedy_next_token_logits")


def grad_sqnorm(g):
    out = torch.empty(1, device="cuda")
    ws = _empty(lib().onn_grad_sqnorm_workspace_floats(i64(g.numel())))
    check(lib().onn_grad_sqnorm(ptr(g), i64(g.numel()), ptr(out), ptr(ws), stream_ptr()), "onn_grad_sqnorm")
    return out


def adam(p, m, v, g, iteration, lr=1e-3, beta1=0.9, beta2=0.999, eps=None, clip_norm=1.0, sqnorm=None,
         grad_scale=1.0, zero_grad=False):
    import numpy as np
    eps = float(np.finfo(np.float32).eps) if eps is None else eps
    bc1 = float(np.float32(1) - np.power(np.float32(beta1), np.float32(iteration)))
    bc2 = float(np.float32(1) - np.power(np.float32(beta2), np.float32(iteration)))
    check(lib().onn_adam(ptr(p), ptr(m), ptr(v), ptr(g), i64(p.numel()), f32(lr), f32(beta1), f32(beta2), f32(eps),
                         f32(bc1), f32(bc2), f32(clip_norm), ptr(sqnorm), f32(grad_scale), int(zero_grad), stream_ptr()), "onn_adam")
