"""Host logic of the sequence-sharded decode on CPU: the shard plan, and the two exchanges as world_size-2 gloo ranks."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def sharded():
    if not os.path.exists(os.path.join(ROOT, "mlops_b200", "lib", "libmlops_attention.so")):
        import __graft_entry__
        __graft_entry__.build()
    from mlops_b200.attention import sharded
    return sharded


@pytest.mark.parametrize("tokens,world", [(262144, 2), (262144, 8), (1 << 20, 8), (4096, 3), (300, 8), (128, 4), (129, 2), (1000, 1)])
def test_plan_covers_the_sequence(sharded, tokens, world):
    plans = sharded.plan_shards(tokens, world)
    groups = (tokens + 127) // 128
    assert len(plans) == min(world, groups)
    assert plans[0].token_first == 0 and plans[-1].token_end == tokens
    closed = 0
    for a, b in zip(plans, plans[1:]):
        assert a.token_end == b.token_first and a.token_end % 128 == 0 and a.extra == 1
    for p in plans:
        n = (p.token_end - p.token_first + 127) // 128
        assert n >= 1 and p.group_first + p.group_count <= n
        assert (p.windows & 1) == (p.rank == 0) and bool(p.windows & 2) == (p.rank == len(plans) - 1)
        closed += p.group_count
    assert plans[-1].extra == 0
    assert closed == max(groups - 2, 0)       # every group but the sink and the open one is some rank's closed group


RANK_SCRIPT = r"""
import os, sys
sys.path.insert(0, os.environ["FBLA_ROOT"])
import numpy as np, torch, torch.distributed as dist
from mlops_b200.attention import sharded
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=2)
rank, rows = dist.get_rank(), 12
rng = np.random.default_rng(5)
mass_all = rng.normal(size=(2, rows)).astype(np.float32); mass_all[1, 3] = -np.inf
part_all = rng.normal(size=(2, rows * sharded.PARTIAL_STRIDE)).astype(np.float32)
gathered = torch.empty(2 * rows)
sharded.exchange_mass(torch.from_numpy(mass_all[rank].copy()), gathered)
assert np.array_equal(gathered.numpy().reshape(2, rows), mass_all)
total = np.log2(np.exp2(gathered.numpy().reshape(2, rows).astype(np.float64)).sum(0))
assert np.allclose(total, np.log2(np.exp2(mass_all.astype(np.float64)).sum(0)))
p = torch.from_numpy(part_all[rank].copy())
sharded.exchange_partial(p)
assert np.allclose(p.numpy(), part_all.sum(0), rtol=1e-6, atol=1e-6)
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_exchanges_two_gloo_ranks(sharded, tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29571", FBLA_ROOT=ROOT)
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
             for r in range(2)]
    outs = [p.communicate(timeout=120)[0].decode() for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in o, o


def test_linked_step_argument_checks_without_a_device(sharded):
    """mlops_fbla_shard_step / mlops_fbla_shard_mailbox_bytes reject bad links before anything is launched."""
    import ctypes
    from mlops_b200.attention import _C
    lib = sharded._lib
    assert lib.mlops_fbla_shard_mailbox_bytes(0, 32) == 0 and lib.mlops_fbla_shard_mailbox_bytes(9, 32) == 0 and lib.mlops_fbla_shard_mailbox_bytes(2, 0) == 0
    one, eight = lib.mlops_fbla_shard_mailbox_bytes(1, 32), lib.mlops_fbla_shard_mailbox_bytes(8, 32)
    assert 0 < one < eight and one % 256 == 0 and eight % 256 == 0
    # 8 ranks x 32 rows: masses 8 x 128 B, sums 8 x 16 896 B, plus this rank's own copies and the flags
    assert eight >= 8 * 32 * 4 + 8 * 32 * 132 * 4 + 32 * 132 * 4
    cfg = _C.Config(1, 32, 8, 4096, 0.0, 0.0, 0, 0, 0, 0, 0, 0, 0)
    cache = _C.Cache(*([0x1000] * 7), None)
    sh = sharded.Shard(1, 10, 3)
    vp = ctypes.c_void_p
    boxes = (ctypes.c_void_p * 2)(0x10000, 0x20000)
    def call(link):
        return lib.mlops_fbla_shard_step(ctypes.byref(cfg), ctypes.byref(sh), ctypes.byref(link), vp(0x1000), ctypes.byref(cache), vp(0x1000), vp(0x1000),
                                         ctypes.c_size_t(1 << 30), None)
    bad_world = sharded.Link(0, 9, ctypes.cast(boxes, ctypes.POINTER(ctypes.c_void_p)), 0)
    assert call(bad_world) == _C.INVALID_VALUE and "world" in _C.last_error()
    bad_rank = sharded.Link(2, 2, ctypes.cast(boxes, ctypes.POINTER(ctypes.c_void_p)), 0)
    assert call(bad_rank) == _C.INVALID_VALUE
    odd = (ctypes.c_void_p * 2)(0x10000, 0x20010)  # the second mailbox is not on a 256-byte boundary
    assert call(sharded.Link(0, 2, ctypes.cast(odd, ctypes.POINTER(ctypes.c_void_p)), 0)) == _C.INVALID_VALUE and "mailbox 1" in _C.last_error()
