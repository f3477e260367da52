"""Work-item interface without a GPU: structure layouts, and that every device entry compiles at run time (NVRTC,
compute_100a) under an executor's own position policy -- the way an executor consumes include/mlops_fbla_items.cuh."""
import ctypes

import pytest

from tests import items_util as iu


def test_structure_layouts():
    assert ctypes.sizeof(iu.Items) == 752 and iu.Items.entry.offset == 24 and iu.Items.args_type.offset == 184
    assert iu.Items.args_bytes.offset == 232 and iu.Items.args.offset == 240 and iu.Items.geom.offset == 496
    assert ctypes.sizeof(iu.Range) == 40
    assert iu.KINDS["CLOSE"] == 1 and iu.KINDS["QKV_CHUNK"] == 12 and iu.ARGS.index("SCRATCH") == 12 and len(iu.ARGS) == 24


ENTRIES = [
    ("fbla::close_item<3, 3>", "fbla_k_prefill", 256), ("fbla::close_item<4, 2>", "fbla_k_prefill", 256), ("fbla::finish_item", "fbla_k_prefill", 256),
    ("fbla::attend_rows_item<3, 3>", "fbla_k_prefill", 256), ("fbla::attend_rows_item<4, 2>", "fbla_k_prefill", 256),
    ("fbla::tc::attend_tc_item<3, 3>", "fbla_k_prefill", 672), ("fbla::tc::attend_tc_item<4, 2>", "fbla_k_prefill", 672),
    ("fbla::coarse_item<3, 3, 4, 2>", "fbla_k_decode", 256), ("fbla::coarse_item<4, 2, 2, 0>", "fbla_k_decode", 256), ("fbla::coarse_item<4, 2, 1, 1>", "fbla_k_decode", 256),
    ("fbla::select_item<4>", "fbla_k_decode", 256), ("fbla::refine_item<3, 3, 4>", "fbla_k_decode", 384), ("fbla::refine_item<4, 2, 2>", "fbla_k_decode", 384),
    ("fbla::merge_item<4>", "fbla_k_decode", 512),
    ("fbla::qkv_token_item<true>", "fbla_k_token", 256), ("fbla::qkv_token_item<false>", "fbla_k_token", 256),
    ("fbla::qkv_chunk_item<true>", "fbla_k_token", 256), ("fbla::qkv_chunk_item<false>", "fbla_k_token", 256),
]


def test_every_entry_compiles_under_an_executor_policy():
    pytest.importorskip("cuda.bindings.nvrtc")
    src = iu.POLICY
    for i, (entry, args_type, threads) in enumerate(ENTRIES):
        call = (f"mlops_fbla::position(item, gridDim.x, 1, 1); __syncthreads(); "
                f"{entry}(*reinterpret_cast<const {args_type} *>(args), reinterpret_cast<unsigned char *>(sm));")
        src += iu.kernel_source(f"k{i}", threads, call)
    ptx = iu.compile_program(src, want_cubin=False)
    text = ptx.decode(errors="replace")
    for i in range(len(ENTRIES)):
        assert f".entry k{i}(" in text
    assert "tcgen05.mma" in text and "cp.async.bulk" in text and "griddepcontrol" not in text  # no dependent-launch waits under an executor


def test_plan_builders_reject_bad_arguments_before_touching_a_device():
    """Validation is the stream calls' own and comes first: a bad call returns -1 with the call's message, no CUDA involved."""
    import os
    from tests import gpu_util as gu
    if not os.path.exists(gu.OURS):
        pytest.skip("library not built")
    lib = ctypes.CDLL(gu.OURS)
    lib.mlops_fbla_last_error.restype = ctypes.c_char_p
    vp = ctypes.c_void_p
    cache = gu.Cache(*([0x1000] * 7), None)
    cfg = gu.Config(1, 4, 2, 0, 0, 0, 1, 4096, 0, 0, 0, 0, 0)
    passes = (iu.Items * 4)()
    # decode_at: odd q_heads / kv_heads
    bad = gu.Config(1, 3, 2, 0, 0, 0, 1, 4096, 0, 0, 0, 0, 0)
    assert lib.mlops_fbla_decode_at_items(ctypes.byref(bad), vp(0x1000), vp(0x1000), ctypes.byref(cache), vp(0x1000), vp(0x1000), ctypes.c_size_t(1 << 30), 0, passes, 4) == -1
    assert b"q_heads" in lib.mlops_fbla_last_error()
    # prefill_at: chunk beyond the capacity
    assert lib.mlops_fbla_prefill_at_items(ctypes.byref(cfg), vp(0x1000), vp(0x1000), 5000, vp(0x1000), vp(0x1000), vp(0x1000), ctypes.byref(cache), vp(0x1000), passes, 4) == -1
    assert b"capacity" in lib.mlops_fbla_last_error()
    # append_at: misaligned k
    assert lib.mlops_fbla_append_at_items(ctypes.byref(cfg), vp(0x1000), vp(0x1002), vp(0x1000), ctypes.byref(cache), passes, 4) == -1
    assert b"boundar" in lib.mlops_fbla_last_error()
    # qkv: a norm weight without its partner
    tok = gu.Token(0x1000, 0x1000, 0x1000, 1024, 768, 768, 0x1000, None, 1e-6, 0x1000, 0.0, 0x1000)
    assert lib.mlops_fbla_qkv_at_items(ctypes.byref(cfg), vp(0x1000), ctypes.byref(tok), ctypes.byref(cache), passes, 4) == -1
    assert b"both or neither" in lib.mlops_fbla_last_error()
    assert lib.mlops_fbla_item_access(passes, 4, 7, 0, None, 0) == -1  # pass out of range
