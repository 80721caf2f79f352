"""Worker of tests/test_dp_gpu.py: one rank of a data-parallel run on real GPUs (launched by
torch.distributed.run).  Each rank steps its slice of the tiny config-2 batch through the
trainer with the NCCL communicator attached -- once with the sharded update (reduce-scatter by
buckets small enough that the arena spans several, Adam on the rank's share, all-gather) and once
with the all-reduce and the whole update on every rank -- and its half of a classifier batch
through the text classifier; rank 0 writes what it ends up with."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(out_path):
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from opennn_b200 import trainer
    from tests.golden.make_golden import CONFIGS, classifier_inputs, CLASSIFIER_CASES, network_inputs
    name = "config2_tiny"
    mode, B, S_in, S_dec, V_in, V_out, E, H, F, L, steps, seed, lo, hi = CONFIGS[name]
    net, params, external, targets = network_inputs(name)
    share = B // world
    first = rank * share
    dec = torch.from_numpy(external[-1][first:first + share]).cuda()
    enc = torch.from_numpy(external[-2][first:first + share]).cuda()
    tgt = torch.from_numpy(targets[first:first + share]).cuda()

    comm = None
    results = {}
    for label, sharded in (("sharded", True), ("replicated", False)):
        t = trainer.Trainer(trainer.TRANSFORMER, S_in, S_dec, V_in, V_out, E, H, F, L, share // 2)   # two micro-batches per rank
        t.set_parameters(params)
        if comm is None:
            comm = trainer.dp_init_from_torch(signature={"parameters": t.parameters_number, "micro_batch": share // 2})
        t.set_dp_options(sharded_update=sharded, bucket_floats=50000)
        t.set_dp(comm, world)
        stats = t.step_device(dec, enc, tgt, update=False)
        gradient = t.get_gradients()
        history = [t.step_device(dec, enc, tgt, update=True) for _ in range(steps)]
        # a step without statistics in between: nothing of the exchange may depend on the read-back
        t.step_device(dec, enc, tgt, update=True, want_statistics=False)
        last = t.step_device(dec, enc, tgt, update=True)
        results[label] = dict(stats=np.array(stats), gradient=gradient, history=np.array(history), params=t.get_parameters(), last=np.array(last),
                              segments=np.array(t.exchange_segments()))
        t.close()

    case = "classifier_tiny"
    cB, cS, cV, cE, cH, hidden, classes, _ = CLASSIFIER_CASES[case]
    _, cparams, ids, ctargets = classifier_inputs(case)
    cshare = cB // world
    c = trainer.TextClassifier(cV, cS, cE, cH, [hidden], classes, cshare)
    c.set_parameters(cparams)
    c.set_dp(comm, world)
    mine = slice(rank * cshare, (rank + 1) * cshare)
    ids_d, targets_d = torch.from_numpy(ids[mine]).cuda(), torch.from_numpy(ctargets[mine]).cuda()
    error, norm = c.step_device(ids_d, targets_d, update=False)
    summed = c.get_gradients()
    losses = [c.step_device(ids_d, targets_d, update=True)[0] for _ in range(3)]
    classifier = dict(error=error, norm=norm, gradient=summed / world, losses=np.array(losses), params=c.get_parameters())
    c.close()

    if rank == 0:
        flat = {f"{label}_{key}": value for label, r in results.items() for key, value in r.items()}
        flat.update({f"classifier_{key}": value for key, value in classifier.items()})
        np.savez(out_path, **flat)
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
