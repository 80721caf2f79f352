"""CPU: the C-ABI library builds for sm_100a, loads without a GPU and exports every symbol
that include/onn_b200.h declares.  No compute call is made here."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(onn_[a-z0-9_]+)\s*\(", text)))


def test_kernel_library_exports_header(built):
    from opennn_b200 import capi
    symbols = declared_symbols("onn_b200.h")
    assert len(symbols) >= 30
    handle = ctypes.CDLL(built["kernels"])
    missing = [s for s in symbols if not hasattr(handle, s)]
    assert not missing, f"declared in onn_b200.h but not exported: {missing}"
    assert sorted(capi.EXPORTS) == symbols, "capi.EXPORTS must list exactly the header's entry points"


def test_status_strings_and_argument_checks(built):
    """Host-side error behaviour needs no GPU: bad arguments are refused before any launch."""
    from opennn_b200 import capi
    L = capi.lib()
    assert L.onn_status_string(0) == b"ok"
    assert L.onn_version() >= 100
    assert L.onn_gemm(None, None) == -1
    assert L.onn_add(None, None, None, ctypes.c_int64(4), ctypes.c_uint32(0), None) == -1
    assert L.onn_layernorm_bwd_workspace_floats(ctypes.c_int64(1000), ctypes.c_int64(512)) > 0
    assert L.onn_gemm_set_mode(7) == -1


def test_host_library_exports_header(built):
    from opennn_b200 import capi, trainer
    symbols = declared_symbols("onn_b200_host.h")
    ctypes.CDLL(built["kernels"], mode=ctypes.RTLD_GLOBAL)
    handle = ctypes.CDLL(built["host"])
    missing = [s for s in symbols if not hasattr(handle, s)]
    assert not missing, f"declared in onn_b200_host.h but not exported: {missing}"
    assert sorted(trainer.HOST_EXPORTS) == symbols


def test_trainer_refuses_without_gpu(built):
    """No CPU fallback: without a CUDA device the host mirror fails loudly."""
    import torch
    if torch.cuda.is_available():
        return
    from opennn_b200 import capi, trainer
    try:
        trainer.Trainer(trainer.TRANSFORMER, 8, 8, 16, 16, 8, 2, 16, 1, 2)
    except capi.OnnError as error:
        assert "no CUDA device" in str(error)
    else:
        raise AssertionError("creating a trainer without a GPU must fail")


def test_reference_side_binding_compiles():
    """oracle/binding_check.cpp defines Normalization3d's two ...Cuda overrides (opennn/layer.h:348-358) with calls into
    the C ABI and is compiled against the reference's own headers.  Needs the OpenNN checkout (OPENNN_REFERENCE, or a
    directory named "reference" beside this repository); skipped where there is none."""
    import shutil
    import subprocess
    import pytest
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    reference = os.environ.get("OPENNN_REFERENCE", os.path.join(os.path.dirname(root), "reference"))
    if not os.path.isdir(os.path.join(reference, "opennn")) or shutil.which("make") is None:
        pytest.skip("no OpenNN checkout here")
    subprocess.run(["make", "-C", os.path.join(root, "oracle"), f"REF={reference}", "binding-check"], check=True, capture_output=True)
