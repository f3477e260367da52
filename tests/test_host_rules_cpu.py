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
def test_the_deal_is_monotone_in_the_token_count(lib, cb):
    """Short rows: by the lengths; long ones: by cost; one window warp per CTA in between. The choice never goes back as
    the rows grow (decode and decode_at of one cache must agree on it, and it is made from a ceiling)."""
    seen = []
    for tokens in list(range(1, 600, 7)) + list(range(600, 70000, 128)) + [131072, 262144, 1 << 20, 1 << 26]:
        deal, _ = split_of(lib, cb, 1, 8, 1, tokens)
        assert deal in (LENGTHS, FIXED, COST)
        seen.append((tokens, deal))
    deals = [d for _, d in seen]
    assert deals == sorted(deals), "the regimes follow one another: lengths, fixed, cost"
    first = {d: min(t for t, x in seen if x == d) for d in (LENGTHS, FIXED, COST)}
    assert first[LENGTHS] == 1
    assert 4000 <= first[FIXED] <= 5500            # about 4 700 tokens
    assert (18000 if cb == 3 else 30000) <= first[COST] <= (23000 if cb == 3 else 37000)
    assert split_of(lib, cb, 1, 8, 1, 131072)[0] == COST and split_of(lib, cb, 8, 8, 1, 16384)[0] == FIXED
    assert split_of(lib, cb, 1, 8, 2, 4096)[0] == LENGTHS


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
