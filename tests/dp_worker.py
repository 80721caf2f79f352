"""Worker of tests/test_dp_gpu.py: one rank of a data-parallel run on real GPUs (launched by
torch.distributed.run).  Each rank steps its slice of the tiny config-2 batch through the
trainer with the NCCL communicator attached; rank 0 writes what it ends up with."""

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
    from tests.golden.make_golden import CONFIGS, network_inputs
    name = "config2_tiny"
    mode, B, S_in, S_dec, V_in, V_out, E, H, F, L, steps, seed, lo, hi = CONFIGS[name]
    net, params, external, targets = network_inputs(name)
    share = B // world
    first = rank * share
    dec = torch.from_numpy(external[-1][first:first + share]).cuda()
    enc = torch.from_numpy(external[-2][first:first + share]).cuda()
    tgt = torch.from_numpy(targets[first:first + share]).cuda()

    t = trainer.Trainer(trainer.TRANSFORMER, S_in, S_dec, V_in, V_out, E, H, F, L, share // 2)   # two micro-batches per rank
    t.set_parameters(params)
    comm = trainer.dp_init_from_torch(signature={"parameters": t.parameters_number, "micro_batch": share // 2})
    t.set_dp(comm, world)
    stats = t.step_device(dec, enc, tgt, update=False)
    gradient = t.get_gradients()
    history = [t.step_device(dec, enc, tgt, update=True) for _ in range(steps)]
    after = t.get_parameters()
    if rank == 0:
        np.savez(out_path, stats=np.array(stats), gradient=gradient, history=np.array(history), params=after)
    t.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
