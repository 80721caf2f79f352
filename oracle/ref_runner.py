"""Runs the reference harness binary (`oracle/_ref/onn_ref_harness`, the UNMODIFIED OpenNN
CPU library built by `oracle/Makefile`) on numpy inputs.

TEST INFRASTRUCTURE ONLY: used by the golden-fixture generator, the tests and the
benchmark's CPU-baseline leg.  The binary is prebuilt; nothing here reads the reference
checkout at run time.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
HARNESS = os.path.join(HERE, "_ref", "onn_ref_harness")
# the same harness built against the reference's own CUDA path (`make -C oracle cuda`): modes transformer_cuda / decoder_cuda
HARNESS_CUDA = os.path.join(HERE, "_ref_cuda", "onn_ref_harness_cuda")


def available() -> bool:
    return os.path.isfile(HARNESS) and os.access(HARNESS, os.X_OK)


def cuda_available() -> bool:
    return os.path.isfile(HARNESS_CUDA) and os.access(HARNESS_CUDA, os.X_OK)


def run(spec: dict, tensors: dict, outputs: list[str], threads: int | None = None, keep: bool = False, cuda: bool = False):
    """Write spec + tensors to a scratch dir, run the harness, read back `outputs`.
    Returns (dict name -> flat float32 array, list of per-step seconds).
    cuda: run the binary built with the reference's CUDA path (its *_cuda modes)."""
    binary = HARNESS_CUDA if cuda else HARNESS
    if not (cuda_available() if cuda else available()):
        raise RuntimeError("reference harness not built: make -C oracle" + (" cuda" if cuda else ""))
    scratch = tempfile.mkdtemp(prefix="onn_ref_")
    try:
        spec = dict(spec)
        if threads is not None:
            spec["threads"] = threads
        with open(os.path.join(scratch, "spec.txt"), "w") as f:
            for key, value in spec.items():
                f.write(f"{key}={value}\n")
        for name, array in tensors.items():
            np.ascontiguousarray(array, dtype=np.float32).tofile(os.path.join(scratch, name + ".bin"))
        env = dict(os.environ)
        if threads is not None:
            env["OMP_NUM_THREADS"] = str(threads)
        subprocess.run([binary, scratch], check=True, env=env)
        result = {}
        for name in outputs:
            path = os.path.join(scratch, name + ".bin")
            if os.path.exists(path):
                result[name] = np.fromfile(path, dtype=np.float32)
        seconds = []
        timing = os.path.join(scratch, "timing.txt")
        if os.path.exists(timing):
            with open(timing) as f:
                seconds = [float(line) for line in f if line.strip()]
        return result, seconds
    finally:
        if not keep:
            shutil.rmtree(scratch, ignore_errors=True)
