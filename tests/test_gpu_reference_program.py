"""The reference's own known-answer program against this library: attention/fbla/tests/test_fbla.cu uses the public C
API only, so oracle/build_ref.sh compiles it UNMODIFIED and links it with mlops_b200/lib/libmlops_attention.a instead
of the reference's library (oracle/_ref/test_fbla_ours; built where the reference tree is mounted, it travels with the
repository's other built files). Its matrix (attention/fbla/tests/test_fbla.cu:1181-1299): decode against its float64
host model for GQA ratios 1 .. 16, contexts up to 262 144 tokens, tau 0 / 1e30 / 1e-30, capacity-padded and strided
("three layers side by side") caches, each twice on a 0xFF-poisoned scratch with bit-equal results; chunked prefill
with the closed groups' bytes against its host packer; host-length calls against CUDA graphs of the device-length
calls, bit for bit; the fused QKV steps; per-row lengths; output layouts -- all from a pool of host threads calling the
API concurrently on one GPU."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROGRAM = os.path.join(ROOT, "oracle", "_ref", "test_fbla_ours")


@pytest.mark.skipif(not os.path.exists(PROGRAM), reason="oracle/_ref/test_fbla_ours was not built (needs the reference tree at build time)")
def test_reference_known_answer_program_passes_on_this_library():
    run = subprocess.run([PROGRAM], capture_output=True, text=True, timeout=1500)
    tail = "\n".join(run.stdout.splitlines()[-40:])
    failed = [line for line in run.stdout.splitlines() if line.startswith("[FAIL]") or " differs " in line]
    assert run.returncode == 0 and "all passed" in run.stdout and not failed, f"{len(failed)} failed:\n" + "\n".join(failed[:20]) + "\n...\n" + tail + run.stderr[-2000:]
    assert run.stdout.count("[PASS]") >= 180
