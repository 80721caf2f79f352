"""GPU: the LayerNorm backward entry point that takes no workspace (onn_layernorm_bwd_static),
for callers that cannot allocate device memory (see include/onn_b200.h).  It must give what
onn_layernorm_bwd gives with a caller-provided workspace, call after call, although every call
reuses the same fixed buffer inside the library.  This file is collected last on purpose: if
it fails, a run that stops at the first failure has already run every other test."""

import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def run_both(capi, rows, E, seed, consumers):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, E, device="cuda", generator=gen) * 3
    gamma = torch.rand(E, device="cuda", generator=gen) + 0.5
    beta = torch.randn(E, device="cuda", generator=gen)
    grads = [torch.randn(rows, E, device="cuda", generator=gen) for _ in range(consumers)]
    y, mean, inv_std, _ = capi.layernorm_fwd(x, gamma, beta)
    extra = grads[1:] + [None, None]
    expected = capi.layernorm_bwd(grads[0], x, mean, inv_std, gamma, dY2=extra[0], dY3=extra[1])

    dx = torch.empty_like(x)
    dgamma = torch.zeros(E, device="cuda")
    dbeta = torch.zeros(E, device="cuda")
    status = capi.lib().onn_layernorm_bwd_static(
        capi.ptr(grads[0]), capi.ptr(extra[0]), capi.ptr(extra[1]), capi.ptr(x), capi.ptr(mean), capi.ptr(inv_std),
        capi.ptr(gamma), capi.ptr(dx), capi.ptr(dgamma), capi.ptr(dbeta), C.c_int64(rows), C.c_int64(E), C.c_uint32(0),
        capi.stream_ptr())
    capi.check(status, "onn_layernorm_bwd_static")
    torch.cuda.synchronize()
    return expected, (dx, dgamma, dbeta)


def test_static_scratch_matches_workspace_entry_point(built):
    from opennn_b200 import capi
    from tests.util import assert_close
    capi.lib()
    # two calls in a row with different sizes: the second must not see anything of the first
    for rows, E, seed, consumers in ((4099, 1024, 1, 2), (777, 256, 2, 1), (4099, 1024, 3, 3)):
        expected, got = run_both(capi, rows, E, seed, consumers)
        for name, a, b in zip(("dx", "dgamma", "dbeta"), got, expected):
            assert_close(a.cpu().numpy(), b.cpu().numpy(), 1e-5, f"{name} (rows {rows}, E {E})")


def test_static_scratch_rejects_rows_wider_than_its_buffer(built):
    from opennn_b200 import capi
    capi.lib()
    E = 2048
    x = torch.zeros(8, E, device="cuda")
    v = torch.zeros(8, device="cuda")
    g = torch.ones(E, device="cuda")
    status = capi.lib().onn_layernorm_bwd_static(
        capi.ptr(x), None, None, capi.ptr(x), capi.ptr(v), capi.ptr(v), capi.ptr(g), capi.ptr(x), capi.ptr(g), capi.ptr(g),
        C.c_int64(8), C.c_int64(E), C.c_uint32(0), capi.stream_ptr())
    assert status == -7, "rows wider than ONN_LAYERNORM_BWD_STATIC_MAX_E must be refused (ONN_ERR_LIMIT)"
    assert capi.lib().onn_status_string(status) == b"size beyond a fixed maximum"
