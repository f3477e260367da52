"""Two real GPUs: the sequence-sharded decode with its exchanges done by the GPUs themselves (mlops_fbla_shard_step,
peer stores + bounded polls over NVLink) against the NCCL-driven step and the one-GPU decode of the whole sequence.
Skipped on a box with one GPU. The two ranks are child processes, one per GPU; a rank leaves only after its last step
has completed on both."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist
    from mlops_b200.attention import sharded
    from tests import datagen
    from tests import gpu_util as gu
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ok = True
        for mode, N, seed in (("3+3", 20000, 5), ("4+2", 9000, 6)):
            q, k, v = datagen.baseline_case(seed, 1, 32, 8, N, outliers=False)
            plan = sharded.plan_shards(N, world)[rank]
            sl = slice(plan.token_first, plan.token_end + plan.extra)
            qd = gu.bf16_tensor(q, dev)
            shard = sharded.encode_shard(gu.bf16_tensor(k[:, :, sl], dev), gu.bf16_tensor(v[:, :, sl], dev), mode, plan)
            want = sharded.decode(qd, shard, dist.group.WORLD).clone()   # the NCCL-driven step
            step = sharded.LinkedDecode(qd, shard, dist.group.WORLD)
            outs = [step().clone() for _ in range(4)]
            torch.cuda.synchronize()
            a, b = (datagen.bf16_to_f32(gu.bits_of(x)).astype(np.float64) for x in (outs[-1], want))
            ok &= step.status() == 0 and all(torch.equal(outs[0], o) for o in outs[1:])
            ok &= bool((np.abs(a - b) <= gu.bf16_ulp(b)).all())            # (the ranks' sums are added in another order there)
            if rank == 0:  # and against the whole sequence in one cache on one GPU
                lib = gu.CLib(gu.OURS)
                single = datagen.bf16_to_f32(gu.bits_of(lib.decode(lib.encode(gu.bf16_tensor(k, dev), gu.bf16_tensor(v, dev), mode), qd))).astype(np.float64)
                ok &= bool((np.abs(a - single) <= 2e-3 * np.abs(single).max() + gu.bf16_ulp(single)).all())
            # every rank holds the same bits
            gathered = [torch.empty_like(outs[-1]) for _ in range(world)]
            dist.all_gather(gathered, outs[-1])
            ok &= all(torch.equal(g, gathered[0]) for g in gathered)
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ret[rank] = int(flag.item())
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_linked_decode_on_two_gpus():
    import torch.multiprocessing as mp
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, 29000 + os.getpid() % 2000, ret), nprocs=world, join=True)
    assert all(ret.get(r) == 1 for r in range(world)), dict(ret)
