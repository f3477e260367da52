"""The decode's arithmetic without its final rounding. The BF16 output of a long-context decode carries up to half an ulp
of rounding (up to 3.9e-3 of the row's largest value), which hides how close the FP32 result is to the float64 model.
The sequence-shard interface returns a row's sums before the division and the rounding (include/mlops_fbla_shard.h:
`partial` = o[128] and l in FP32, relative to the row's mass), and one shard that holds the whole cache runs exactly
the kernels of mlops_fbla_decode; so o / l is the decode's unrounded output. It must agree with the oracle's float64
decode to 2e-4 of the largest output, a tenth of the tolerance the BF16 outputs are held to."""
import numpy as np
import pytest
import torch

from tests import datagen
from tests import gpu_util as gu

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["3+3", "4+2"])
@pytest.mark.parametrize("B,QH,KH,N,seed,outliers", [(1, 16, 8, 4096, 1001, True),      # BASELINE configs[0]
                                                     (2, 32, 8, 16384, 1002, True),     # two rows of configs[1]
                                                     (1, 32, 8, 131072, 1003, False)])  # the metric's 128K context
def test_unrounded_decode_output_against_float64_model(oracle, mode, B, QH, KH, N, seed, outliers):
    from mlops_b200.attention import sharded
    q, k, v = datagen.baseline_case(seed, B, QH, KH, N, outliers=outliers)
    qd, kd, vd = gu.bf16_tensor(q), gu.bf16_tensor(k), gu.bf16_tensor(v)
    shard = sharded.encode_shard(kd, vd, mode, sharded.plan_shards(N, 1)[0])
    rows = B * QH
    mass = sharded.local_mass(qd, shard)
    total = torch.empty(rows, dtype=torch.float32, device="cuda")
    sharded.total_mass(mass, 1, rows, total)
    partial = sharded.local_partial(qd, shard, total).view(rows, sharded.PARTIAL_STRIDE).double().cpu().numpy()
    got = (partial[:, :128] / partial[:, 128:129]).reshape(B, QH, 128)
    want = oracle.decode(q, oracle.encode(k, v, mode))
    rel = np.abs(got - want).max() / np.abs(want).max()
    print(f"\n[parity] unrounded decode B{B} {QH}q/{KH}kv ctx{N} {mode}: max|ours_fp32 - oracle_f64| / max|oracle| = {rel:.2e}")
    assert rel <= 2e-4, rel
