"""GPU, two ranks over NCCL: the data-parallel step (slices of the batch, global active-token
count, gradient exchange by buckets from inside back-propagation) against the single-GPU step
and the reference's golden loss trajectory -- with the sharded update (reduce-scatter, clip +
Adam on each rank's share of the arena, all-gather of the parameters) and with the all-reduce
and the whole update on every rank -- and the data-parallel step of the text classifier against
its single-GPU step.  Skipped on boxes with fewer than two GPUs."""

import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from tests.golden.make_golden import CONFIGS, network_inputs
from tests.util import TOL, assert_close, errors, golden

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
    t.step_device(dec, enc, tgt, update=True, want_statistics=False)
    last = t.step_device(dec, enc, tgt, update=True)
    after = t.get_parameters()
    t.close()

    g = golden(name)
    for label in ("sharded", "replicated"):
        assert dp[f"{label}_stats"][2] == stats[2], "both must count the active tokens of the whole batch"
        assert abs(dp[f"{label}_stats"][0] - stats[0]) <= 1e-5 * abs(stats[0])
        assert_close(dp[f"{label}_gradient"], gradient, 1e-4, "gradient, 2 GPUs x 2 micro-batches vs 1 GPU")
        for step in range(steps):
            assert abs(dp[f"{label}_history"][step][0] - g["loss"][2 * step]) <= TOL * abs(g["loss"][2 * step])
            assert abs(dp[f"{label}_history"][step][0] - history[step][0]) <= 1e-4 * abs(history[step][0])
            assert abs(dp[f"{label}_history"][step][3] - history[step][3]) <= 1e-4 * abs(history[step][3]), "gradient norm"
        assert abs(dp[f"{label}_last"][0] - last[0]) <= 1e-4 * abs(last[0])
        # a gradient that is zero in exact arithmetic (the key biases) is rounding noise that depends on how the batch was
        # cut; Adam turns it into small steps of either sign, so the element-wise bound is Adam's step and the L2 bound 1e-3
        _, l2_err = errors(dp[f"{label}_params"], after)
        assert l2_err <= TOL, f"parameters after {steps + 2} steps, {label} vs 1 GPU: l2-rel {l2_err:.2e}"
        assert np.abs(dp[f"{label}_params"] - after).max() <= 2.2e-3 * (steps + 2)
    # the two data-parallel modes reduce the same per-rank gradients (up to the order of floating-point atomics): their
    # parameters agree as closely as two runs of one mode do
    # (with work items by counter the order of the floating-point atomics also changes from run to run, and Adam turns the
    # sign of a gradient that is rounding noise into a step: L2 as two runs of one mode, single elements within Adam's steps)
    _, l2_err = errors(dp["sharded_params"], dp["replicated_params"])
    assert l2_err <= 1e-4, f"parameters, sharded update vs update on every rank: l2-rel {l2_err:.2e}"
    assert np.abs(dp["sharded_params"] - dp["replicated_params"]).max() <= 2.2e-3 * (steps + 2)
    assert dp["sharded_segments"] > 2, "the exchanging micro-batch of the sharded update is replayed from graph segments"

    # text classifier: the two ranks' averaged gradient and their steps against one GPU on the whole batch
    from tests.golden.make_golden import CLASSIFIER_CASES, classifier_inputs
    cB, cS, cV, cE, cH, hidden, classes, _ = CLASSIFIER_CASES["classifier_tiny"]
    _, cparams, ids, ctargets = classifier_inputs("classifier_tiny")
    c = trainer.TextClassifier(cV, cS, cE, cH, [hidden], classes, cB)
    c.set_parameters(cparams)
    ids_d, targets_d = torch.from_numpy(ids).cuda(), torch.from_numpy(ctargets).cuda()
    error, norm = c.step_device(ids_d, targets_d, update=False)
    whole = c.get_gradients()
    losses = [c.step_device(ids_d, targets_d, update=True)[0] for _ in range(3)]
    cafter = c.get_parameters()
    c.close()
    assert abs(float(dp["classifier_error"]) - error) <= 1e-5 * abs(error)
    assert abs(float(dp["classifier_norm"]) - norm) <= 1e-3 * abs(norm)
    assert_close(dp["classifier_gradient"], whole, TOL, "classifier gradient, average of 2 ranks vs the whole batch")
    for a, b in zip(dp["classifier_losses"], losses):
        assert abs(a - b) <= TOL * abs(b)
    assert np.abs(dp["classifier_params"] - cafter).max() <= 2.2e-3 * 3
