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
    ("fbla::coarse_item<3, 3, 4>", "fbla_k_decode", 384), ("fbla::coarse_item<4, 2, 2>", "fbla_k_decode", 384), ("fbla::coarse_item<4, 2, 1>", "fbla_k_decode", 384),
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
