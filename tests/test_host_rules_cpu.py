"""Host-side rules of the decode that need no GPU: how the coarse pass's work is dealt (fbla_k_decode_split), checked
through the built library, and the bench's accounting of algorithmic bytes."""
import ctypes
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS, FIXED, COST = 0, 1, 2  # FBLA_K_DEAL_*


@pytest.fixture(scope="module")
def lib():
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import __graft_entry__
    path = os.path.join(ROOT, "mlops_b200", "lib", "libmlops_attention.so")
    if not os.path.exists(path):
        __graft_entry__.build()
    return ctypes.CDLL(path)


def split_of(lib, cb, batch, kv_heads, vg, tokens):
    deal, fold = ctypes.c_int(-1), ctypes.c_int(-1)
    lib.fbla_k_decode_split_of(cb, batch, kv_heads, vg, ctypes.c_longlong(tokens), ctypes.byref(deal), ctypes.byref(fold))
    return deal.value, fold.value


@pytest.mark.parametrize("cb", [3, 4])
def test_the_deal_follows_the_groups_a_warp_would_stream(lib, cb):
    """Short rows: by the lengths. Beyond: seven + one or by cost, whichever leaves a streaming warp fewer whole groups
    (counted for 148 CTAs of eight warps), with 5 % against the deal by cost."""
    for tokens in list(range(1, 4000, 97)):
        assert split_of(lib, cb, 1, 8, 1, tokens)[0] == LENGTHS
    assert split_of(lib, cb, 256, 8, 1, 512)[0] == LENGTHS and split_of(lib, cb, 1, 8, 2, 4096)[0] == LENGTHS
    for tokens in list(range(6000, 70000, 128)) + [131072, 262144, 1 << 20, 1 << 26]:
        for batch in (1, 8, 64):
            deal, _ = split_of(lib, cb, batch, 8, 1, tokens)
            heads, S = batch * 8, (tokens + 127) // 128 - 2
            fixed = -(-heads * S // (148 * 7))
            cost = -(-(8 * heads * S + 4 * heads * 16) // (8 * 148 * 8))
            assert deal == (COST if 21 * cost < 20 * fixed else FIXED), (tokens, batch, fixed, cost)
    assert split_of(lib, cb, 1, 8, 1, 131072)[0] == COST    # 7 groups per warp instead of 8
    assert split_of(lib, cb, 8, 8, 1, 16384)[0] == FIXED    # 8 either way
    assert split_of(lib, cb, 64, 8, 1, 65280)[0] == COST


def test_rows_are_folded_per_cta_for_few_heads_only(lib):
    assert split_of(lib, 3, 1, 8, 1, 131072)[1] == 1      # 8 virtual heads, long rows
    assert split_of(lib, 4, 8, 8, 1, 16384)[1] == 0       # 64 virtual heads
    assert split_of(lib, 3, 1, 8, 1, 2048)[1] == 0        # split by the lengths: never folded
    assert split_of(lib, 4, 4, 8, 1, 65536)[1] == 1       # 32 virtual heads: the last folded size
    assert split_of(lib, 4, 4, 8, 2, 65536)[1] == 0


def test_bench_accounts_the_bytes_the_way_the_reference_bench_does():
    """Algorithmic bytes of a decode: per closed (KV head, group) 8 coarse records + 1 KiB of metadata, 512 B per BF16
    window token, 3 072 B per refined (KV head, sub-block) (attention/fbla/bench/bench_fbla.cu:136-141)."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import bench
    assert set(bench.NCU_TRAFFIC) <= set(bench.WORKLOADS) and set(bench.SUBS) <= set(bench.WORKLOADS)
    assert bench.WORKLOADS["decode_128k"]["tokens"] == 131072 and bench.WORKLOADS["decode_128k"]["mode"] == "3+3"
    total, parts = bench.decode_bytes(dict(batch=1, kv_heads=8, tokens=131072, mode="3+3"), 0.0)
    groups = 131072 // 128 - 2
    assert parts["coarse_and_meta"] == 8 * groups * (8 * 1536 + 1024)
    assert parts["bf16_windows"] == 8 * 256 * 512 and total == parts["coarse_and_meta"] + parts["bf16_windows"]
    total, parts = bench.decode_bytes(dict(batch=8, kv_heads=8, tokens=16384, mode="4+2"), 0.5)
    assert parts["coarse_and_meta"] == 64 * 126 * (8 * 2048 + 1024) and parts["refine"] == 0.5 * 64 * 126 * 8 * 3072


def test_reference_arm_prints_the_contract_line_without_a_gpu():
    """`bench.py --impl reference` is the oracle's port of the reference's host model on the host cores: it needs no GPU,
    and its one JSON line carries the keys the measurement contract names."""
    import json
    import subprocess
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [l for l in run.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "decode_tokens_per_s" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["config"]["tokens"] == 131072 and d["config"]["mode"] == "3+3" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == dict(value=d["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)
