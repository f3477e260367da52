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


def _shards_of(q, k, v, N, world, mode):
    from mlops_b200.attention import sharded
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    out = []
    for p in sharded.plan_shards(N, world):
        sl = slice(p.token_first, p.token_end + p.extra)
        out.append(sharded.encode_shard(kd[:, :, sl].contiguous(), vd[:, :, sl].contiguous(), mode, p))
    return qd, out


def test_linked_step_one_rank_equals_the_step_of_separate_calls():
    """mlops_fbla_shard_step with a world of one (its stores and polls all go to its own mailbox), eagerly and replayed
    from one CUDA graph, against the same passes driven call by call."""
    from mlops_b200.attention import sharded
    q, k, v = datagen.baseline_case(78, 1, 8, 2, 6000)
    qd, (shard,) = _shards_of(q, k, v, 6000, 1, "3+3")
    want = sharded.decode(qd, shard).clone()
    step = sharded.LinkedDecode(qd, shard)
    for _ in range(3):
        assert torch.equal(step(), want)
    assert step.status() == 0
    eager = sharded.LinkedDecode(qd, shard, graph=False)
    assert torch.equal(eager(), want) and eager.status() == 0


@pytest.mark.parametrize("mode", ["3+3", "4+2"])
def test_linked_step_with_the_peer_data_already_delivered(mode):
    """Two shards, one GPU, no kernel ever waits for another launch: the second rank's masses and sums are computed with
    the call-by-call interface and placed in rank 0's mailbox, stamped with the step number, before rank 0's step is
    enqueued, so its polls succeed at once. Rank 0's output must be the combination of both shards."""
    from mlops_b200.attention import sharded
    import ctypes
    QH, N = 8, 5000
    q, k, v = datagen.uneven_case(11, 1, QH, 2, N)
    qd, shards = _shards_of(q, k, v, N, 2, mode)
    rows = QH
    masses = torch.cat([sharded.local_mass(qd, s, tau=1e-3).clone() for s in shards])
    total = torch.empty(rows, dtype=torch.float32, device="cuda")
    sharded.total_mass(masses, 2, rows, total)
    partials = [sharded.local_partial(qd, s, total, tau=1e-3).clone() for s in shards]
    want = sharded.combine(partials[0] + partials[1], qd).clone()
    # rank 0's mailbox, laid out as fbla_k_mailbox_of(2, rows): 16 B epoch, status to 256, mass flags at 256, sum flags at 512, ...
    nbytes = sharded._lib.mlops_fbla_shard_mailbox_bytes(2, rows)
    up = lambda n: (n + 255) // 256 * 256
    off_mass_in = 768
    off_part_in = off_mass_in + up(2 * rows * 4) + 2 * up(rows * 4)
    box0 = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    box1 = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")  # where rank 0's stores for its peer land; nobody reads it
    box0[256:264].view(torch.int32)[1] = 1                         # mass flag of rank 1: step 1
    box0[512:520].view(torch.int32)[1] = 1                         # sum flag of rank 1
    box0[off_mass_in:off_mass_in + 2 * rows * 4].view(torch.float32)[rows:] = masses[rows:]
    box0[off_part_in:off_part_in + 2 * rows * 132 * 4].view(torch.float32)[rows * 132:] = partials[1]
    torch.cuda.synchronize()
    step = sharded.LinkedDecode(qd, shards[0], tau=1e-3, mailboxes=[box0.data_ptr(), box1.data_ptr()], rank=0, graph=False, wait_polls=20000)
    torch.cuda.synchronize()
    assert step.status() == 0
    a, b = datagen.bf16_to_f32(gu.bits_of(step.out)).astype(np.float64), datagen.bf16_to_f32(gu.bits_of(want)).astype(np.float64)
    assert (np.abs(a - b) <= gu.bf16_ulp(b)).all()  # (the sums are added in rank order here, as one tensor sum there)
    # what rank 0 stored for its peer: its own masses and sums in slot 0 of the peer's mailbox, stamped 1
    assert box1[256:264].view(torch.int32)[0].item() == 1 and box1[512:520].view(torch.int32)[0].item() == 1
    assert torch.equal(box1[off_mass_in:off_mass_in + rows * 4].view(torch.float32), masses[:rows])
    sent = box1[off_part_in:off_part_in + rows * 132 * 4].view(torch.float32).view(rows, 132)
    assert torch.equal(sent[:, :129], partials[0].view(rows, 132)[:, :129])  # o[128] and l; the row's last three floats are padding


def test_linked_step_gives_up_on_a_silent_peer():
    """A peer that never writes: the bounded poll runs out (here after 2 000 polls of 64 ns), the step still completes, the
    status word names the exchange and the silent rank, and the output is NaN instead of a plausible number. (The waiting
    kernel polls a word in global memory that nothing sets; no copy is in flight and nothing faults.)"""
    from mlops_b200.attention import sharded
    q, k, v = datagen.baseline_case(79, 1, 8, 2, 3000)
    qd, shards = _shards_of(q, k, v, 3000, 2, "4+2")
    nbytes = sharded._lib.mlops_fbla_shard_mailbox_bytes(2, 8)
    box0 = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    box1 = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    step = sharded.LinkedDecode(qd, shards[0], mailboxes=[box0.data_ptr(), box1.data_ptr()], rank=0, graph=False, wait_polls=2000)
    torch.cuda.synchronize()
    assert step.status() == 1 + 16 * 1  # the mass exchange, rank 1
    assert torch.isnan(step.out.float()).all()
    # the context is healthy: an ordinary decode afterwards works
    lib = gu.CLib(gu.OURS)
    c = lib.encode(gu.bf16_tensor(k), gu.bf16_tensor(v), "4+2")
    assert torch.isfinite(lib.decode(c, qd).float()).all()
