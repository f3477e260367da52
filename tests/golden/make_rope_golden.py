"""Generates tests/golden/rope_golden.npz for the fused QKV step by IMPORTING the reference's own Python code (CPU only):

  * positional/python/mlops/positional/rope.py  rope_frequencies  (float64 inverse frequencies, the attention factor)

and, for the rotation and the RMSNorm, whose only CPU statement in the reference is the formula (transformers'
apply_rotary_pos_emb and Qwen3RMSNorm, cited by attention/include/mlops_fbla.h:169-172), a float64 evaluation of that
formula on seeded inputs. Run in the build container:  python tests/golden/make_rope_golden.py <path to the reference tree>
"""
import importlib.util
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests import datagen  # noqa: E402


def main(ref_root):
    for name in ("mlops", "mlops.positional", "mlops.positional._C"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["mlops.positional"]._C = sys.modules["mlops.positional._C"]
    spec = importlib.util.spec_from_file_location("mlops.positional.rope", os.path.join(ref_root, "positional", "python", "mlops", "positional", "rope.py"))
    rope = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rope)
    out = {}
    for theta in (1e4, 1e6):
        inv, att = rope.rope_frequencies(128, theta)
        out[f"inv_freq_{int(theta)}"] = inv.numpy().astype(np.float64)
        out[f"att_{int(theta)}"] = np.float64(att)
    # float64 formula on seeded BF16 inputs: y = rms_norm(x) * w (optional), then x cos + rotate_half(x) sin
    rng = np.random.default_rng(77)
    x = datagen.to_bf16_bits(rng.standard_normal((6, 128), dtype=np.float32) * 2.0)
    w = datagen.to_bf16_bits(rng.standard_normal(128, dtype=np.float32) * 0.5)
    pos = np.array([0, 1, 127, 4096, 70001, 1000003], np.int64)
    xf, wf = datagen.bf16_to_f32(x).astype(np.float64), datagen.bf16_to_f32(w).astype(np.float64)
    inv = out["inv_freq_1000000"]
    ang = pos[:, None].astype(np.float64) * inv[None, :]
    c, s = np.cos(ang), np.sin(ang)

    def rotate(v):
        return np.concatenate([v[:, :64] * c - v[:, 64:] * s, v[:, 64:] * c + v[:, :64] * s], 1)

    normed = xf / np.sqrt((xf * xf).mean(1, keepdims=True) + 1e-6) * wf
    out["x_bits"], out["w_bits"], out["positions"] = x, w, pos
    out["rope_only"] = rotate(xf)
    out["norm_rope"] = rotate(normed)
    path = os.path.join(HERE, "rope_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["MLOPS_REFERENCE_ROOT"])
