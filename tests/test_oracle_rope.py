"""The oracle's restatement of the fused QKV step (RMSNorm + rotary embedding) against tests/golden/rope_golden.npz:
the reference's own float64 inverse frequencies, and the float64 formula of the norm and the rotation on seeded inputs."""
import os

import numpy as np

from tests import datagen

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_golden.npz"))


def test_frequency_table_matches_reference_frequencies(oracle):
    for theta in (1e4, 1e6):
        inv = G[f"inv_freq_{int(theta)}"]
        f = oracle.rope_freq(theta).astype(np.float64)
        want = inv / (2 * np.pi)
        assert np.abs((f[:, 0] + f[:, 1]) - want).max() <= 1e-15 * want.max() + 1e-22  # (fh, fl) carries f to ~2^-48
        g = np.mod(65536.0 * want, 1.0)
        d = np.abs((f[:, 2] + f[:, 3]) - g)
        assert np.minimum(d, 1 - d).max() < 1e-9
        assert G[f"att_{int(theta)}"] == 1.0


def _ulp_ok(got_bits, want64, ulps=1.0):
    got = datagen.bf16_to_f32(got_bits).astype(np.float64)
    ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(want64), 1e-30))) - 7)
    return (np.abs(got - want64) <= ulps * ulp + 1e-30).all()


def test_rotation_matches_float64_formula(oracle):
    f = oracle.rope_freq(1e6)
    got = oracle.norm_rope(G["x_bits"], None, 0.0, G["positions"], f)
    # one rounding to BF16 of an FP32 evaluation: within 0.51 ulp of the float64 value (phases are exact to ~2^-24 turns)
    assert _ulp_ok(got, G["rope_only"], 0.51)


def test_norm_and_rotation_match_float64_formula(oracle):
    f = oracle.rope_freq(1e6)
    got = oracle.norm_rope(G["x_bits"], G["w_bits"], 1e-6, G["positions"], f)
    # two intermediate BF16 roundings (x r, then times w) by definition, then the rotation's: within 2 BF16 ulps of the
    # unrounded float64 formula at the scale of the pair
    want = G["norm_rope"]
    pair = np.maximum(np.abs(want[:, :64]), np.abs(want[:, 64:]))
    scale = np.concatenate([pair, pair], 1)
    got64 = datagen.bf16_to_f32(got).astype(np.float64)
    assert (np.abs(got64 - want) <= 3 * 2.0 ** (np.floor(np.log2(scale)) - 7)).all()


def test_position_zero_is_identity(oracle):
    f = oracle.rope_freq(1e6)
    got = oracle.norm_rope(G["x_bits"][:1], None, 0.0, 0, f)
    assert np.array_equal(got, G["x_bits"][:1])
