"""Sequence-sharded decode (include/mlops_fbla_shard.h): the shards of one long sequence, here all on one GPU and run
one after the other (the exchanges replaced by a concatenation and a sum), against the oracle's decode of the whole
sequence and against the single-cache decode."""
import numpy as np
import pytest
import torch

from tests import datagen
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["3+3", "4+2"])
@pytest.mark.parametrize("QH,KH,N,world,seed,gen", [(8, 2, 3000, 2, 3, "uneven_case"), (32, 8, 5000, 3, 1003, "baseline_case"),
                                                    (4, 2, 2048, 5, 5, "uneven_case"), (16, 8, 700, 8, 7, "uneven_case"),
                                                    (8, 2, 1500, 1, 9, "uneven_case")])
def test_sharded_decode_matches_oracle(oracle, mode, QH, KH, N, world, seed, gen):
    from mlops_b200.attention import sharded
    q, k, v = getattr(datagen, gen)(seed, 1, QH, KH, N)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    plans = sharded.plan_shards(N, world)
    assert plans[0].token_first == 0 and plans[-1].token_end == N
    shards = []
    for p in plans:
        sl = slice(p.token_first, p.token_end + p.extra)
        shards.append(sharded.encode_shard(kd[:, :, sl].contiguous(), vd[:, :, sl].contiguous(), mode, p))
    rows = QH
    masses = torch.cat([sharded.local_mass(qd, s, tau=1e-3).clone() for s in shards])
    total = torch.empty(rows, dtype=torch.float32, device="cuda")
    sharded.total_mass(masses, len(shards), rows, total)
    partial = sum(sharded.local_partial(qd, s, total, tau=1e-3).clone() for s in shards)
    out = sharded.combine(partial, qd)
    torch.cuda.synchronize()
    want = oracle.decode(q, oracle.encode(k, v, mode), tau=1e-3)
    gu.check_close(gu.bits_of(out), want, f"{mode} {world} shards of {N}")
    lib = gu.CLib(gu.OURS)
    single = datagen.bf16_to_f32(gu.bits_of(lib.decode(lib.encode(kd, vd, mode), qd, tau=1e-3))).astype(np.float64)
    got = datagen.bf16_to_f32(gu.bits_of(out)).astype(np.float64)
    assert (np.abs(got - single) <= 2e-3 * np.abs(single).max() + gu.bf16_ulp(single)).all()


def test_graphed_decode_equals_eager_decode():
    """The step replayed from CUDA graphs (one rank: no exchange) gives the eager step's bits, call after call."""
    from mlops_b200.attention import sharded
    q, k, v = datagen.baseline_case(77, 1, 8, 2, 5000)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    shard = sharded.encode_shard(kd, vd, "4+2", sharded.plan_shards(5000, 1)[0])
    want = sharded.decode(qd, shard).clone()
    step = sharded.GraphedDecode(qd, shard)
    for _ in range(3):
        assert torch.equal(step(), want)
