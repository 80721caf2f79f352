"""GPU, two ranks over NCCL: the data-parallel step (slices of the batch, global active-token
count, bucketed gradient all-reduce, clip + Adam on every rank) against the single-GPU step
and the reference's golden loss trajectory.  Skipped on boxes with fewer than two GPUs."""

import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from tests.golden.make_golden import CONFIGS, network_inputs
from tests.util import TOL, assert_close, golden

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_match_one(built):
    from opennn_b200 import trainer
    name = "config2_tiny"
    steps = CONFIGS[name][10]
    with tempfile.TemporaryDirectory() as out_dir:
        out_path = os.path.join(out_dir, "dp.npz")
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29611", os.path.join(ROOT, "tests", "dp_worker.py"), out_path],
                       check=True, env=env, timeout=600)
        dp = dict(np.load(out_path))

    mode, B, S_in, S_dec, V_in, V_out, E, H, F, L, _, seed, lo, hi = CONFIGS[name]
    net, params, external, targets = network_inputs(name)
    t = trainer.Trainer(trainer.TRANSFORMER, S_in, S_dec, V_in, V_out, E, H, F, L, B)
    t.set_parameters(params)
    dec, enc, tgt = (torch.from_numpy(x).cuda() for x in (external[-1], external[-2], targets))
    stats = t.step_device(dec, enc, tgt, update=False)
    gradient = t.get_gradients()
    history = [t.step_device(dec, enc, tgt, update=True) for _ in range(steps)]
    t.close()

    g = golden(name)
    assert dp["stats"][2] == stats[2], "both must count the active tokens of the whole batch"
    assert abs(dp["stats"][0] - stats[0]) <= 1e-5 * abs(stats[0])
    assert_close(dp["gradient"], gradient, 1e-4, "gradient, 2 GPUs x 2 micro-batches vs 1 GPU")
    for step in range(steps):
        assert abs(dp["history"][step][0] - g["loss"][2 * step]) <= TOL * abs(g["loss"][2 * step])
        assert abs(dp["history"][step][0] - history[step][0]) <= 1e-4 * abs(history[step][0])
