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
# Sharded update: reduce-scatter by buckets, clip + Adam on each rank's share, all-gather
# ---------------------------------------------------------------------------------------

def _sharded_rank_main(rank, world, init_file, out_dir, bucket_floats):
    """What a data-parallel step that updates does (opennn_b200/host/driver_abi.cpp, sharded_update), restated with the
    numpy oracle over gloo: per bucket of the fixed grid the ranks' gradients are summed and each rank keeps its part
    (gloo has no reduce-scatter for CPU tensors: an all-reduce followed by taking the own part gives the same values),
    the squared norms of the own parts are summed over ranks, clip + Adam run on the own parts with moments that exist
    for those parts only, and an all-gather per bucket rebuilds the parameter arena on every rank."""
    from opennn_b200 import trainer
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    net, params, external, targets = network_inputs("tiny_encdec_odd")
    batch = targets.shape[0]
    bounds = np.linspace(0, batch, world + 1).astype(int)
    lo, hi = bounds[rank], bounds[rank + 1]
    shard = {k: v[lo:hi] for k, v in external.items()}
    t = O.token_index(targets[lo:hi])
    count = torch.tensor([float(((t > 0) & (t < net.layers[-1]["out"])).sum())])
    dist.all_reduce(count)

    total, bucket, parts = trainer.shard_layout(params.size, world, bucket_floats)
    arena = np.zeros(total, dtype=np.float32)                     # the arena rounded up; the slack stays zero
    arena[:params.size] = params
    gradient = np.zeros(total, dtype=np.float32)
    own_m, own_v = np.zeros(total // world, dtype=np.float32), np.zeros(total // world, dtype=np.float32)
    steps = 3
    for step in range(steps):
        probabilities = net.forward(arena[:params.size], shard)
        gradient[:params.size] = net.backward(arena[:params.size], O.ce3d_output_gradients(probabilities, targets[lo:hi], active_count=int(count.item())))
        own_gradient = np.zeros(total // world, dtype=np.float32)
        for low, part in reversed(parts):                          # back-propagation finishes the top of the arena first
            reduced = torch.from_numpy(gradient[low:low + part * world].copy())
            dist.all_reduce(reduced)
            own_gradient[low // world:low // world + part] = reduced.numpy()[rank * part:(rank + 1) * part]
        square = torch.tensor([float(np.sum(own_gradient.astype(np.float64) ** 2))], dtype=torch.float64)
        dist.all_reduce(square)
        norm = np.float32(np.sqrt(square.item()))
        for low, part in parts:
            own = slice(low // world, low // world + part)
            mine = arena[low + rank * part:low + (rank + 1) * part]          # a view: updated in place
            O.adam_update(mine, own_gradient[own], own_m[own], own_v[own], step + 2, norm=norm)
            gathered = [torch.empty(part) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(mine.copy()))
            arena[low:low + part * world] = torch.cat(gathered).numpy()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), params=arena[:params.size], slack=arena[params.size:])
    dist.destroy_process_group()


def test_sharded_update_gives_the_replicated_step():
    """Three steps of the sharded update on two ranks, with buckets small enough that the arena spans several and the
    last one is ragged, against three whole-batch steps on one replica: same parameters to 1e-6, identical on both ranks,
    and the slack the arena was rounded up by stays zero."""
    world = 2
    with tempfile.TemporaryDirectory() as out_dir:
        init_file = os.path.join(out_dir, "rendezvous")
        mp.spawn(_sharded_rank_main, args=(world, init_file, out_dir, 3000), nprocs=world, join=True)
        ranks = [np.load(os.path.join(out_dir, f"rank{r}.npz")) for r in range(world)]
    net, params, external, targets = network_inputs("tiny_encdec_odd")
    arena, m, v, iteration = params.copy(), np.zeros_like(params), np.zeros_like(params), 1
    for _ in range(3):
        _, _, _, iteration = net.train_step(arena, m, v, iteration, external, targets)
    for r in ranks:
        assert np.abs(r["params"] - arena).max() <= 1e-6 * max(1.0, np.abs(arena).max())
        assert not r["slack"].any()
    assert np.array_equal(ranks[0]["params"], ranks[1]["params"]), "replicas must stay identical"


def test_shard_layout_covers_the_arena_in_aligned_parts():
    from opennn_b200 import trainer
    for parameters, world, bucket in [(276712, 2, 50000), (276712, 8, 16 << 20), (1000, 3, 100), (64, 4, 16), (17, 2, 1)]:
        total, size, parts = trainer.shard_layout(parameters, world, bucket)
        assert total >= parameters and total - parameters < 4 * world and total % (4 * world) == 0
        assert size % (4 * world) == 0
        covered = 0
        for low, part in parts:
            assert low == covered and part % 4 == 0 and low % (4 * world) == 0
            covered += part * world
        assert covered == total
        assert sum(part for _, part in parts) == total // world


def _classifier_rank_main(rank, world, init_file, out_dir):
    """The data-parallel rule of the text classifier (opennn_b200/host/classifier_abi.cpp): every rank back-propagates
    its own samples with the loss averaged over ITS samples, the gradient arenas are summed, the update divides by the
    number of ranks."""
    from tests.golden.make_golden import classifier_inputs
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    net, params, ids, targets = classifier_inputs("classifier_tiny")
    share = ids.shape[0] // world
    mine = slice(rank * share, (rank + 1) * share)
    probabilities = net.forward(params, {-1: ids[mine]})
    gradient = net.backward(params, O.ce2d_output_gradients(probabilities, targets[mine]))
    error = torch.tensor([float(O.ce2d_error(probabilities, targets[mine]))])
    reduced = torch.from_numpy(gradient.copy())
    dist.all_reduce(reduced)
    dist.all_reduce(error)
    averaged = (reduced.numpy() / np.float32(world)).astype(np.float32)
    arena, m, v = params.copy(), np.zeros_like(params), np.zeros_like(params)
    O.adam_update(arena, averaged, m, v, 2)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), gradient=averaged, params=arena, error=error.numpy() / world)
    dist.destroy_process_group()


def test_classifier_ranks_reproduce_the_whole_batch_step():
    from tests.golden.make_golden import classifier_inputs
    world = 2
    with tempfile.TemporaryDirectory() as out_dir:
        init_file = os.path.join(out_dir, "rendezvous")
        mp.spawn(_classifier_rank_main, args=(world, init_file, out_dir), nprocs=world, join=True)
        ranks = [np.load(os.path.join(out_dir, f"rank{r}.npz")) for r in range(world)]
    net, params, ids, targets = classifier_inputs("classifier_tiny")
    assert ids.shape[0] % world == 0
    probabilities = net.forward(params, {-1: ids})
    gradient = net.backward(params, O.ce2d_output_gradients(probabilities, targets))
    arena, m, v = params.copy(), np.zeros_like(params), np.zeros_like(params)
    O.adam_update(arena, gradient, m, v, 2)
    for r in ranks:
        assert abs(float(r["error"][0]) - float(O.ce2d_error(probabilities, targets))) <= 1e-6
        assert np.abs(r["gradient"] - gradient).max() <= 1e-5 * np.abs(gradient).max()
        assert np.abs(r["params"] - arena).max() <= 2e-6


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
