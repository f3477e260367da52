"""Seeded synthetic inputs for the parity tests, the golden fixtures and the bench (numpy only, so the same bytes
are produced on every machine). BF16 tensors are carried as uint16 bit patterns."""
import numpy as np


def to_bf16_bits(x):
    """float32 array -> BF16 bit patterns (round to nearest even)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def baseline_case(seed, batch, q_heads, kv_heads, tokens, outliers=True, q_rows=None):
    """The benchmark distribution: q, k, v i.i.d. N(0,1) rounded to BF16; with `outliers`, 4 of the 128 channels of
    every (batch, KV head) are scaled x8 in K and V. q is [batch, q_heads, 128], or [batch, q_heads, q_rows, 128]."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((batch, kv_heads, tokens, 128), dtype=np.float32)
    v = rng.standard_normal((batch, kv_heads, tokens, 128), dtype=np.float32)
    qshape = (batch, q_heads, 128) if q_rows is None else (batch, q_heads, q_rows, 128)
    q = rng.standard_normal(qshape, dtype=np.float32)
    if outliers:
        for b in range(batch):
            for h in range(kv_heads):
                ch = rng.permutation(128)[:4]
                k[b, h, :, ch] *= 8.0
                v[b, h, :, ch] *= 8.0
    return to_bf16_bits(q), to_bf16_bits(k), to_bf16_bits(v)


def uneven_case(seed, batch, q_heads, kv_heads, tokens, q_rows=None):
    """The distribution the reference's own tests use (attention/python/tests/test_attention.py:89-95,
    attention/fbla/tests/test_fbla.cu:100-112): K with uneven per-channel ranges and an offset of 3 on every 7th
    channel, V ~ N(0,1), q ~ 1.5 N(0,1)."""
    rng = np.random.default_rng(seed)
    chan = (0.2 + 1.5 * rng.random(128)).astype(np.float32)
    off = ((np.arange(128) % 7) == 0).astype(np.float32) * 3.0
    k = rng.standard_normal((batch, kv_heads, tokens, 128), dtype=np.float32) * chan + off
    v = rng.standard_normal((batch, kv_heads, tokens, 128), dtype=np.float32)
    qshape = (batch, q_heads, 128) if q_rows is None else (batch, q_heads, q_rows, 128)
    q = 1.5 * rng.standard_normal(qshape, dtype=np.float32)
    return to_bf16_bits(q), to_bf16_bits(k), to_bf16_bits(v)


def edge_group(seed):
    """[128, 128] BF16 group with hard quantizer channels: constant, all-negative, zero-minimum, huge range, tiny
    range, all-zero, very small."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((128, 128), dtype=np.float32)
    x[:, 0] = 1.25                      # constant: step 0
    x[:, 1] = -np.abs(x[:, 1]) - 0.5    # all negative
    x[:, 2] = np.abs(x[:, 2]); x[5, 2] = 0.0      # minimum exactly 0
    x[:, 3] *= 1e4                      # huge range
    x[:, 4] = 3.0 + 1e-3 * x[:, 4]      # tiny range relative to the offset
    x[:, 5] = 0.0                       # all zero
    x[:, 6] *= 1e-20                    # very small magnitudes (steps below 1e-30 are clamped by the reference's Python twin only)
    x[:, 7] = -x[:, 7] * 8.0            # outlier channel
    x[:, 8] = np.where(np.arange(128) % 2 == 0, 1.0, -1.0)  # two-valued
    return to_bf16_bits(x)
