"""CPU, two gloo ranks: the data-parallel rule the GPU driver implements
(opennn_b200/host/driver_abi.cpp) restated with the numpy oracle.  Each rank takes a contiguous
slice of the batch, scales its loss gradient by the active-token count of the WHOLE batch
(summed across ranks first), and the ranks' parameter gradients are summed: the result must be
the gradient of the whole batch, and Adam on it must give the same parameters on every rank."""

import os
import tempfile

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import opennn_oracle as O
from tests.golden.make_golden import network_inputs


def _rank_main(rank, world, init_file, out_dir):
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    net, params, external, targets = network_inputs("tiny_encdec_odd")
    batch = targets.shape[0]
    # ragged split on purpose (3 samples over 2 ranks): slices need not be equal
    bounds = np.linspace(0, batch, world + 1).astype(int)
    lo, hi = bounds[rank], bounds[rank + 1]
    shard = {k: v[lo:hi] for k, v in external.items()}
    shard_targets = targets[lo:hi]

    t = O.token_index(shard_targets)
    count = torch.tensor([float(((t > 0) & (t < net.layers[-1]["out"])).sum())])
    dist.all_reduce(count)                                   # (1) global active-token count

    probabilities = net.forward(params, shard)
    gradient = net.backward(params, O.ce3d_output_gradients(probabilities, shard_targets, active_count=int(count.item())))
    reduced = torch.from_numpy(gradient.copy())
    dist.all_reduce(reduced)                                 # (2) sum of the parameter gradients

    arena, m, v = params.copy(), np.zeros_like(params), np.zeros_like(params)
    O.adam_update(arena, reduced.numpy(), m, v, 2)           # (3) clip + Adam on the reduced gradient, every rank
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), gradient=reduced.numpy(), params=arena, count=count.numpy())
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_whole_batch_step():
    world = 2
    with tempfile.TemporaryDirectory() as out_dir:
        init_file = os.path.join(out_dir, "rendezvous")
        mp.spawn(_rank_main, args=(world, init_file, out_dir), nprocs=world, join=True)
        ranks = [np.load(os.path.join(out_dir, f"rank{r}.npz")) for r in range(world)]

    net, params, external, targets = network_inputs("tiny_encdec_odd")
    probabilities = net.forward(params, external)
    _, _, count = O.ce3d_error(probabilities, targets)
    gradient = net.backward(params, O.ce3d_output_gradients(probabilities, targets))
    arena, m, v = params.copy(), np.zeros_like(params), np.zeros_like(params)
    O.adam_update(arena, gradient, m, v, 2)

    for r in ranks:
        assert int(r["count"][0]) == count
        scale = np.abs(gradient).max()
        assert np.abs(r["gradient"] - gradient).max() <= 1e-5 * scale
        assert np.abs(r["params"] - arena).max() <= 2e-6
    assert np.array_equal(ranks[0]["params"], ranks[1]["params"]), "replicas must stay identical"


# ---------------------------------------------------------------------------------------
# Failure detection, on the host: no GPU, no NCCL, nothing faults or hangs
# ---------------------------------------------------------------------------------------

def _rendezvous_main(rank, world, init_file, out_dir, scenario):
    import datetime
    from opennn_b200 import trainer
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    outcome = "ok"
    try:
        if scenario == "missing" and rank == 1:
            outcome = "left before the rendezvous"                 # a rank that exits between steps and never joins
        else:
            parameters = 276712 if not (scenario == "mismatch" and rank == 1) else 276704
            trainer.dp_check_replicas({"parameters": parameters, "micro_batch": 8}, timeout_s=3.0)
    except trainer.DpRendezvousError as error:
        outcome = f"refused: {error}"
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(outcome)
    if scenario != "missing":
        dist.destroy_process_group()


def _run_rendezvous(scenario):
    world = 2
    with tempfile.TemporaryDirectory() as out_dir:
        init_file = os.path.join(out_dir, "rendezvous")
        mp.spawn(_rendezvous_main, args=(world, init_file, out_dir, scenario), nprocs=world, join=True)
        return [open(os.path.join(out_dir, f"rank{r}.txt")).read() for r in range(world)]


def test_replicas_that_agree_may_start():
    assert _run_rendezvous("agree") == ["ok", "ok"]


def test_mismatched_parameter_arena_is_refused_on_every_rank_before_any_launch():
    outcomes = _run_rendezvous("mismatch")
    assert all(o.startswith("refused") and "replica 1 differs" in o for o in outcomes), outcomes


def test_missing_rank_ends_the_rendezvous_with_a_timeout_not_a_hang():
    outcomes = _run_rendezvous("missing")
    assert outcomes[1] == "left before the rendezvous"
    assert outcomes[0].startswith("refused") and "[1] did not join" in outcomes[0], outcomes


def test_shard_batch_gives_every_rank_an_equal_contiguous_slice():
    from opennn_b200 import trainer
    ids = np.arange(24).reshape(8, 3)
    parts = [trainer.shard_batch([ids, None], rank, 4) for rank in range(4)]
    assert all(p[1] is None for p in parts)
    assert np.array_equal(np.concatenate([p[0] for p in parts]), ids)
    assert all(p[0].shape[0] == 2 for p in parts)
    try:
        trainer.shard_batch([ids], 0, 3)
        raise AssertionError("a batch that does not divide must be refused")
    except ValueError:
        pass
