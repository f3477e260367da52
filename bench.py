"""Benchmark of the FBLA hot path on B200: compressed-KV decode (headline) and causal prefill.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

The headline line (default workload, `decode_128k`) is the configuration BASELINE.json's metric is quoted on: one decode
step -- one new token -- of batch 1, 32 query heads / 8 KV heads, head_dim 128, over 131 072 cached tokens in 3+3 mode,
seeded BF16 N(0,1) inputs, softmax scale 1/sqrt(128), default tau; the cache was written by the library itself
(quantize-on-write). The same JSON line carries sub-records (`sub`) for the other configurations, each with its own
`ms_per_step`, `e2e` and `roofline`: the 4+2 format at 128K, configs[1] (batch 8 x 16 384, 4+2), configs[3] (causal
prefill batch 4 x 8 192, TFLOP/s) and configs[4] (mixed serving decode, batch 64, ragged 1K..64K contexts).

Timing: after W >= 3 warm-up steps, blocks of exactly K steps between two CUDA events on the launching stream (with a
barrier + synchronize on both sides), repeated until at least half a second has been timed; `ms_per_step` is the median
block. Every step alternates between two copies of the cache that together exceed the 126 MB L2. `value` has its inputs
resident in HBM; `e2e` is the same step through `mlops_b200.attention` with q in pinned host memory and the output
copied back, every step. The decode's four passes are also timed one by one (separate launches) to name the dominant
kernel; `ref_gpu` is the reference's own CUDA library (oracle/_ref, when built) on the same cache; `cpu_baseline` a
bounded sample of the oracle's port of the reference's host-side float64 model on this machine's cores.

N > 1 (torchrun, one rank per GPU): the SAME job split over the ranks (strong scaling) -- the 8 KV heads of the headline
decode are dealt to the ranks, each with its heads' cache; no data-path collective is needed (NCCL carries the barrier
and the max over ranks). Sub-records: configs[1] and configs[4] by KV head, configs[3] by (batch row, KV head), and
configs[2]'s sequence split of one 262 144-token context with its two small exchanges.
`--impl reference` times the reference's host-side path (the oracle port) on the host cores, same configuration.
"""
import argparse
import ctypes
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC, UNIT = "decode_tokens_per_s", "tokens/s"
WORKLOADS = {
    "decode_128k": dict(kind="decode", batch=1, q_heads=32, kv_heads=8, tokens=131072, mode="3+3", seed=1003, outliers=False,
                        name="decode B1 32q/8kv ctx131072 3+3 (the metric's 128K context)"),
    "decode_128k_4p2": dict(kind="decode", batch=1, q_heads=32, kv_heads=8, tokens=131072, mode="4+2", seed=1003, outliers=False,
                            name="decode B1 32q/8kv ctx131072 4+2 (the metric's 128K context)"),
    "decode_4k": dict(kind="decode", batch=1, q_heads=16, kv_heads=8, tokens=4096, mode="3+3", seed=1001, outliers=True,
                      name="decode B1 16q/8kv ctx4096 3+3 (BASELINE configs[0])"),
    "decode_b8": dict(kind="decode", batch=8, q_heads=32, kv_heads=8, tokens=16384, mode="4+2", seed=1002, outliers=True,
                      name="decode B8 32q/8kv ctx16384 4+2 (BASELINE configs[1])"),
    "serving_b64": dict(kind="serving", batch=64, q_heads=32, kv_heads=8, lo=1024, hi=65536, mode="3+3", seed=1005,
                        name="serving decode B64 32q/8kv 3+3, contexts U[1024, 65536], 256-token pages (BASELINE configs[4])"),
    "prefill_b4": dict(kind="prefill", batch=4, q_heads=32, kv_heads=8, tokens=8192, mode="4+2", seed=1004,
                       name="causal prefill B4 S8192 32q/8kv 4+2 (BASELINE configs[3])"),
    "prefill_b1": dict(kind="prefill", batch=1, q_heads=32, kv_heads=8, tokens=8192, mode="4+2", seed=1004,
                       name="causal prefill B1 S8192 32q/8kv 4+2 (one sequence of BASELINE configs[3]; for profiler captures)"),
    "seqsplit_256k": dict(kind="seqsplit", tokens=262144, name="sequence-split decode B1 32q/8kv ctx262144 3+3 (BASELINE configs[2])"),
    "seqsplit_1m": dict(kind="seqsplit", tokens=1 << 20, name="sequence-split decode B1 32q/8kv ctx1048576 3+3 (BASELINE configs[2])"),
}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the workload's dominant kernel, from the ncu captures summarised
# under profiles/ (1 GPU); reported with their source, never as a measurement of the run that prints them
NCU_TRAFFIC = {
    "decode_128k": dict(kernel="coarse_kernel<3,3,4,2>", bytes=113223424, file="profiles/decode_b1_ctx128k_3p3_launches.md"),
    "decode_b8": dict(kernel="refine_kernel<4,2,4>", bytes=164004352, file="profiles/decode_b8_ctx16k_4p2_launches.md"),
}
SUBS = ["decode_128k_4p2", "decode_b8", "prefill_b4", "serving_b64"]
MIN_TIMED_S = 0.5


def peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def hbm_peak():
    p = peaks()
    return (p["hbm_gbs"], "measured") if "hbm_gbs" in p else (6650.0, "fallback")


def bf16(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


class Dist:
    """rank / world of this process, NCCL for the barrier and the max over ranks"""

    def __init__(self):
        import torch
        self.rank, self.world, self.local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, values):
        import torch
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while a timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if not self.nv:
            return
        nv = self.nv
        names = {nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown", nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap"}
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def result(self):
        self.stop_flag = True
        self.join(timeout=1.0)
        return dict(sm_mhz=float(np.median(self.samples)) if self.samples else None, sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons),
                    samples=len(self.samples))


def timed_blocks(D, step, steps, warmup, sample_clocks=False):
    """Warm-up, then blocks of exactly `steps` calls of step(i) between two events, until MIN_TIMED_S has been timed.
    Returns (median ms per step over the blocks, max over ranks), the number of blocks and the clock record."""
    import torch
    stream = torch.cuda.current_stream()
    n = 0
    for _ in range(max(warmup, 3)):
        step(n); n += 1
    sampler = ClockSampler(D.local) if sample_clocks else None
    D.barrier()
    if sampler:
        sampler.start()
    per_step, total = [], 0.0
    while (not per_step or total < MIN_TIMED_S * 1000.0) and len(per_step) < 400:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        D.barrier()
        e0.record(stream)
        for _ in range(steps):
            step(n); n += 1
        e1.record(stream)
        D.barrier()
        ms = D.max([e0.elapsed_time(e1)])[0]  # (every rank sees the same total, so all leave the loop together)
        per_step.append(ms / steps)
        total += ms
    clocks = sampler.result() if sampler else None
    return float(np.median(per_step)), len(per_step), clocks


# ---- decode -----------------------------------------------------------------------------------------------------------------
def decode_bytes(cfg, share, kv_heads=None):
    """Bytes one decode must move (the reference bench's accounting, attention/fbla/bench/bench_fbla.cu:136-141): coarse
    records + 1 KiB metadata of every closed group, the BF16 sink and open tokens (K and V), and coarse + fine records
    of the share of closed sub-blocks that some query of the KV head refines."""
    cb, fb = (3, 3) if cfg["mode"] == "3+3" else (4, 2)
    heads = cfg["batch"] * (cfg["kv_heads"] if kv_heads is None else kv_heads)
    groups = (cfg["tokens"] + 127) // 128
    closed = max(groups - 2, 0)
    open_tokens = cfg["tokens"] - 128 * (groups - 1)
    rc, rf = 2 * cb * 256, 2 * fb * 256
    coarse = heads * closed * (8 * rc + 1024)
    windows = heads * (128 + open_tokens) * 128 * 2 * 2
    refine = share * heads * closed * 8 * (rc + rf)
    return coarse + windows + refine, dict(coarse_and_meta=coarse, bf16_windows=windows, refine=refine)


def decode_plan(_C, cfg_struct, length, qd, cache_struct, out, scratch):
    """The decode's four passes as the plan interface returns them (include/mlops_fbla_items.h): their argument blob is what
    the per-pass launcher takes."""
    from tests import items_util as iu
    lib = _C.lib
    passes = (iu.Items * 4)()
    vp = ctypes.c_void_p
    lib.mlops_fbla_decode_at_items.restype = ctypes.c_int
    n = lib.mlops_fbla_decode_at_items(ctypes.byref(cfg_struct), vp(length.data_ptr()), vp(qd.data_ptr()), ctypes.byref(cache_struct), vp(out.data_ptr()),
                                       vp(scratch.data_ptr()), ctypes.c_size_t(scratch.numel()), 0, passes, 4)
    if n != 4:
        raise RuntimeError(_C.last_error())
    return passes


def time_passes(D, _C, passes, reps=30):
    """Each pass alone (ordinary launches, in order so that every pass finds its inputs), µs per launch."""
    import torch
    lib = _C.lib
    lib.fbla_k_decode_pass_launch.restype = ctypes.c_int
    stream = torch.cuda.current_stream()
    sp = ctypes.c_void_p(stream.cuda_stream)
    times = [[] for _ in range(4)]
    for _ in range(reps):
        for p in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            rc = lib.fbla_k_decode_pass_launch(ctypes.byref(passes[p].args), p, sp)
            e1.record(stream)
            if rc:
                raise RuntimeError(f"pass {p}: CUDA error {rc}")
            torch.cuda.synchronize()
            times[p].append(e0.elapsed_time(e1) * 1000.0)
    return [float(np.median(t[3:])) for t in times]


def refined_share(scratch, vheads, closed_blocks):
    """Fraction of closed (virtual head, sub-block) pairs the select pass listed. The refine pass leaves the total at the end
    of its item_off array, which sits just before the 256-byte status block that ends the scratch."""
    import torch
    up = lambda n: (n + 255) // 256 * 256
    off = scratch.numel() - 256 - up((vheads + 1) * 4) + vheads * 4
    total = int(scratch[off:off + 4].view(torch.int32).item())
    return total / max(1, closed_blocks)


def run_decode(D, cfg, args, headline):
    """One decode workload; with world > 1 the KV heads are dealt to the ranks (each rank: its heads of every batch row)."""
    import torch
    from mlops_b200 import attention
    from mlops_b200.attention import _C
    from tests import datagen

    B, QH, KH, N = cfg["batch"], cfg["q_heads"], cfg["kv_heads"], cfg["tokens"]
    world = min(D.world, KH)
    if D.rank >= world:  # more ranks than KV heads: the surplus ranks only take part in the barriers
        def idle(i):
            pass
        ms, blocks, _ = timed_blocks(D, idle, args.steps, args.warmup)
        timed_blocks(D, idle, args.steps, 3)
        return None
    kh0, kh1 = KH * D.rank // world, KH * (D.rank + 1) // world
    g = QH // KH
    q, k, v = datagen.baseline_case(cfg["seed"], B, QH, KH, N, outliers=cfg["outliers"])
    q, k, v = q[:, kh0 * g:kh1 * g], k[:, kh0:kh1], v[:, kh0:kh1]  # this rank's heads
    qh, kh = (kh1 - kh0) * g, kh1 - kh0
    q_host = bf16(q).pin_memory()
    qd = q_host.to(D.dev)
    kd, vd = bf16(k).to(D.dev), bf16(v).to(D.dev)
    copies = [attention.encode(kd, vd, cfg["mode"]) for _ in range(2)]  # two copies alternated: together larger than L2
    del kd, vd
    c0 = copies[0]
    cs = _C.Config(B, qh, kh, c0.tokens, 0.0, 0.0, c0.format, c0.capacity, 0, 0, 0, 0, 0)
    nbytes = _C.lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(cs))
    scratch = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=D.dev)
    out = torch.empty_like(qd)
    caches = [_C.Cache(c.coarse.data_ptr(), c.fine.data_ptr(), c.meta.data_ptr(), c.sink_k.data_ptr(), c.sink_v.data_ptr(), c.open_k.data_ptr(),
                       c.open_v.data_ptr(), None) for c in copies]
    stream = torch.cuda.current_stream()

    def step(i):
        st = _C.lib.mlops_fbla_decode(ctypes.byref(cs), qd.data_ptr(), ctypes.byref(caches[i & 1]), out.data_ptr(), scratch.data_ptr(), nbytes,
                                      ctypes.c_void_p(stream.cuda_stream))
        if st:
            raise RuntimeError(_C.last_error())

    ms, blocks, clocks = timed_blocks(D, step, args.steps, args.warmup, sample_clocks=True)
    status = scratch[-256:].view(torch.int32)[:2].tolist()
    if status[0]:
        raise RuntimeError(f"a bounded wait gave up: status {status}")
    vheads = B * kh * max(1, g // 4)
    closed_blocks = vheads * max((N + 127) // 128 - 2, 0) * 8
    share = refined_share(scratch, vheads, closed_blocks)

    # ---- end to end through the Python interface: host q -> device, decode, output -> host, every step -----------------
    out_host = torch.empty(q_host.shape, dtype=torch.bfloat16).pin_memory()

    def step_e2e(i):
        o = attention.decode(q_host.to(D.dev, non_blocking=True), copies[i & 1])
        out_host.copy_(o, non_blocking=True)

    ms_e2e, _, _ = timed_blocks(D, step_e2e, args.steps, 3)

    # ---- the passes one by one, and the reference's CUDA library on the same cache (rank 0 of a 1-GPU run) ----------------
    pass_us = ref_us = None
    if D.world == 1:
        length = torch.tensor([N], dtype=torch.int32, device=D.dev)
        cs_at = _C.Config(B, qh, kh, 0, 0.0, 0.0, c0.format, c0.capacity, 0, 0, 0, 0, 0)
        passes = decode_plan(_C, cs_at, length, qd, caches[0], out, scratch)
        step(0)
        torch.cuda.synchronize()
        pass_us = time_passes(D, _C, passes)
        ref_us = ref_gpu_decode(cfg, copies, qd)

    abytes, parts = decode_bytes(cfg, share)
    peak, peak_kind = hbm_peak()
    rec = dict(ms_per_step=ms, blocks=blocks, clocks=clocks, share=share, ms_e2e=ms_e2e, h2d=q_host.numel() * 2 * world, d2h=out_host.numel() * 2 * world,
               abytes=abytes, parts=parts, peak=peak, peak_kind=peak_kind, pass_us=pass_us, ref_us=ref_us, world=world)
    return rec


def ref_gpu_decode(cfg, copies, qd, reps=40):
    """µs per decode of the reference's own CUDA library (built for sm_100 into oracle/_ref by oracle/build_ref.sh) on
    the cache this library wrote -- the cache bytes are the reference's format bit for bit. None when it was not built."""
    import torch
    from tests import gpu_util as gu
    if not os.path.exists(gu.REF):
        return None
    ref = gu.CLib(gu.REF)
    cs = [dict(coarse=c.coarse, fine=c.fine, meta=c.meta, sink_k=c.sink_k, sink_v=c.sink_v, open_k=c.open_k, open_v=c.open_v, tokens=c.tokens,
               capacity=c.capacity, mode=cfg["mode"], batch=c.meta.shape[0], kv_heads=c.meta.shape[1]) for c in copies]
    scratch = ref.scratch(cs[0], qd.shape[1])
    for i in range(5):
        ref.decode(cs[i & 1], qd, scratch=scratch)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        ref.decode(cs[i & 1], qd, scratch=scratch)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / reps


def decode_record(cfg, rec, n_gpus):
    """The JSON fields of one decode workload from run_decode's measurements."""
    per_step = rec["ms_per_step"] * 1e-3
    achieved = rec["abytes"] / per_step / 1e9
    peak = rec["peak"] * rec["world"]
    # DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum): not measured in this run --
    # a profiler cannot run inside the timed program -- but taken from the ncu capture of this workload on one GPU
    captured = NCU_TRAFFIC.get(cfg.get("key")) if n_gpus == 1 else None
    roof = dict(bound="hbm", achieved=achieved, peak=peak, unit="GB/s", frac=achieved / peak, traffic=captured["bytes"] if captured else None,
                traffic_source=(f"ncu capture of {captured['kernel']} on this workload, one launch, not this run: {captured['file']}" if captured
                                else "not captured for this workload; ncu captures of other workloads are summarised under profiles/"),
                peak_kind=rec["peak_kind"] + (f", x {rec['world']} GPUs" if rec["world"] > 1 else ""),
                kernel="decode call: coarse, select, refine, merge", algorithmic_bytes=rec["abytes"], bytes_parts=rec["parts"])
    if rec["pass_us"]:
        names = ["coarse_kernel", "select_kernel", "refine_kernel", "merge_kernel"]
        us = rec["pass_us"]
        bytes_of = [rec["parts"]["coarse_and_meta"] + rec["parts"]["bf16_windows"], None, rec["parts"]["refine"], None]
        top = int(np.argmax(us))
        roof["passes_us"] = dict(zip(names, us))
        roof["dominant_kernel"] = dict(name=names[top], us=us[top], share_of_passes=us[top] / sum(us))
        if bytes_of[top]:
            roof["dominant_kernel"].update(algorithmic_bytes=bytes_of[top], achieved=bytes_of[top] / (us[top] * 1e-6) / 1e9,
                                           frac=bytes_of[top] / (us[top] * 1e-6) / 1e9 / rec["peak"])
    out = dict(metric=METRIC, value=cfg["batch"] / per_step, unit=UNIT, ms_per_step=rec["ms_per_step"], blocks=rec["blocks"],
               config=dict(workload=cfg["name"], l2="two cache copies alternated, together larger than L2", refined_share=rec["share"],
                           sharding=("KV heads over %d GPUs, no exchange" % rec["world"]) if n_gpus > 1 else "one GPU",
                           **{k: cfg[k] for k in ("batch", "q_heads", "kv_heads", "tokens", "mode")}),
               e2e=dict(value=cfg["batch"] / (rec["ms_e2e"] * 1e-3), unit=UNIT, h2d_bytes_per_step=rec["h2d"], d2h_bytes_per_step=rec["d2h"]),
               roofline=roof, dtype="u8")
    if rec["ref_us"]:
        out["ref_gpu"] = dict(us_per_step=rec["ref_us"], speedup=rec["ref_us"] / (rec["ms_per_step"] * 1000.0),
                              what="the reference's CUDA library (its DP4A kernels compiled for sm_100), same GPU, same cache, cache resident")
    return out


# ---- serving decode (configs[4]) ---------------------------------------------------------------------------------------------
def run_serving(D, cfg, args):
    """Batch 64, ragged contexts: per-row device lengths (length_stride 1) over a cache laid out in whole 256-token pages.
    world > 1: the KV heads are dealt to the ranks. Tokens are seeded N(0,1) drawn on the device."""
    import torch
    from mlops_b200 import attention
    from mlops_b200.attention import _C

    B, QH, KH, mode = cfg["batch"], cfg["q_heads"], cfg["kv_heads"], cfg["mode"]
    world = min(D.world, KH)
    if D.rank >= world:
        def idle(i):
            pass
        timed_blocks(D, idle, args.steps, args.warmup)
        return None
    kh = KH * (D.rank + 1) // world - KH * D.rank // world
    qh = kh * (QH // KH)
    lengths = np.random.default_rng(cfg["seed"]).integers(cfg["lo"], cfg["hi"], size=B, endpoint=True).astype(np.int32)
    cap = -(-int(lengths.max()) // 256) * 256
    gen = torch.Generator(device=D.dev)
    gen.manual_seed(cfg["seed"] + 31 * D.rank)
    cache = attention.empty(B, kh, cap, mode, device=D.dev)
    fmt = cache.format
    for b, n in enumerate(lengths):  # every row filled to its own length through a one-row view of the cache
        kk = torch.randn((1, kh, int(n), 128), generator=gen, device=D.dev, dtype=torch.float32).to(torch.bfloat16)
        vv = torch.randn((1, kh, int(n), 128), generator=gen, device=D.dev, dtype=torch.float32).to(torch.bfloat16)
        row = attention.FBLACache(cache.coarse[b:b + 1], cache.fine[b:b + 1], cache.meta[b:b + 1], cache.sink_k[b:b + 1], cache.sink_v[b:b + 1],
                                  cache.open_k[b:b + 1], cache.open_v[b:b + 1], 0, cap, fmt)
        attention.append(row, kk, vv)
    q_host = torch.randn((B, qh, 128), generator=torch.Generator().manual_seed(cfg["seed"] + 1)).to(torch.bfloat16).pin_memory()
    qd = q_host.to(D.dev)
    ld = torch.from_numpy(lengths).to(D.dev)
    cs = _C.Config(B, qh, kh, 0, 0.0, 0.0, fmt, cap, 0, 0, 0, 0, 1)
    lay = _C.Config(B, qh, kh, cap, 0.0, 0.0, fmt, cap, 0, 0, 0, 0, 0)
    nbytes = _C.lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(lay))
    scratch = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=D.dev)
    out = torch.empty_like(qd)
    kc = _C.Cache(cache.coarse.data_ptr(), cache.fine.data_ptr(), cache.meta.data_ptr(), cache.sink_k.data_ptr(), cache.sink_v.data_ptr(),
                  cache.open_k.data_ptr(), cache.open_v.data_ptr(), None)
    stream = torch.cuda.current_stream()
    out_host = torch.empty(q_host.shape, dtype=torch.bfloat16).pin_memory()

    def step(i, q_in=None, o=None):
        st = _C.lib.mlops_fbla_decode_at(ctypes.byref(cs), ld.data_ptr(), (qd if q_in is None else q_in).data_ptr(), ctypes.byref(kc),
                                         (out if o is None else o).data_ptr(), scratch.data_ptr(), nbytes, ctypes.c_void_p(stream.cuda_stream))
        if st:
            raise RuntimeError(_C.last_error())

    ms, blocks, clocks = timed_blocks(D, step, args.steps, args.warmup)  # (the cache itself, ~0.8 GB per KV head, exceeds L2)
    vheads = B * kh
    closed_blocks = int(sum(max((int(n) + 127) // 128 - 2, 0) for n in lengths)) * kh * 8
    share = refined_share(scratch, vheads, closed_blocks)

    def step_e2e(i):  # the device-length call through the C ABI with host q and output (the Python interface has no per-row lengths)
        dq = q_host.to(D.dev, non_blocking=True)
        step(i, dq, out)
        out_host.copy_(out, non_blocking=True)

    ms_e2e, _, _ = timed_blocks(D, step_e2e, args.steps, 3)
    rc, rf = 1536, 1536
    coarse = sum(max((int(n) + 127) // 128 - 2, 0) for n in lengths) * KH * (8 * rc + 1024)
    windows = sum(128 + int(n) - 128 * ((int(n) + 127) // 128 - 1) for n in lengths) * KH * 128 * 2 * 2
    refine = share * closed_blocks / kh * KH * (rc + rf)
    peak, peak_kind = hbm_peak()
    abytes = coarse + windows + refine
    achieved = abytes / (ms * 1e-3) / 1e9
    return dict(metric=METRIC, value=B / (ms * 1e-3), unit=UNIT, ms_per_step=ms, blocks=blocks,
                config=dict(workload=cfg["name"], l2="the cache (~0.8 GB per KV head) exceeds L2", refined_share=share, batch=B, q_heads=QH, kv_heads=KH,
                            mode=mode, lengths=dict(min=int(lengths.min()), max=int(lengths.max()), mean=float(lengths.mean())), capacity=cap,
                            layout="per-row device lengths (length_stride 1); affine units, two group units per 256-token page",
                            sharding=("KV heads over %d GPUs, no exchange" % world) if D.world > 1 else "one GPU"),
                e2e=dict(value=B / (ms_e2e * 1e-3), unit=UNIT, h2d_bytes_per_step=q_host.numel() * 2 * world, d2h_bytes_per_step=out_host.numel() * 2 * world),
                roofline=dict(bound="hbm", achieved=achieved, peak=peak * world, unit="GB/s", frac=achieved / (peak * world), traffic=None,
                              peak_kind=peak_kind, kernel="decode_at call: coarse, select, refine, merge", algorithmic_bytes=abytes,
                              bytes_parts=dict(coarse_and_meta=coarse, bf16_windows=windows, refine=refine)),
                dtype="u8")


# ---- prefill (configs[3]) ----------------------------------------------------------------------------------------------------
def run_prefill(D, cfg, args):
    """Causal prefill of whole sequences into an empty cache: quantize-on-write of the chunk's groups, attention over the
    compressed cache on tensor cores, window update. world > 1: the (batch row, KV head) units are dealt to the ranks.
    FLOPs: 4 * 128 per (query, attended key) pair."""
    import torch
    from mlops_b200 import attention
    from tests import datagen

    B, QH, KH, S, mode = cfg["batch"], cfg["q_heads"], cfg["kv_heads"], cfg["tokens"], cfg["mode"]
    units = B * KH
    world = min(D.world, units)
    if D.rank >= world:
        def idle(i):
            pass
        timed_blocks(D, idle, min(args.steps, 10), 3)
        timed_blocks(D, idle, min(args.steps, 10), 3)
        return None
    g = QH // KH
    if world == 1:
        q, k, v = datagen.baseline_case(cfg["seed"], B, QH, KH, S, q_rows=S, outliers=True)
        nb, kv = B, KH
    else:
        # this rank's (batch row, KV head) units as a batch of single-KV-head sequences: the units are independent, so the
        # ranks' calls together are the whole problem (unit b KH + h = batch row b, KV head h)
        u0, u1 = units * D.rank // world, units * (D.rank + 1) // world
        rows = [datagen.baseline_case(cfg["seed"] + 7919 * u, 1, g, 1, S, q_rows=S, outliers=True) for u in range(u0, u1)]
        q, k, v = (np.concatenate([r[i] for r in rows]) for i in range(3))
        nb, kv = u1 - u0, 1
    host = [bf16(x).pin_memory() for x in (q, k, v)]
    qd, kd, vd = [x.to(D.dev) for x in host]
    cache = attention.empty(nb, kv, S, mode, device=D.dev)
    steps = min(args.steps, 10)

    def step(i):
        cache.tokens = 0  # the same buffers, refilled from the start
        return attention.prefill(qd, kd, vd, cache)

    ms, blocks, clocks = timed_blocks(D, step, steps, min(args.warmup, 5))
    out_host = torch.empty(qd.shape, dtype=torch.bfloat16).pin_memory()
    # end to end: a three-stage pipeline over batch rows and steps. The inputs come from pinned host memory row by row on a
    # copy stream into one of two sets of device buffers (so the next step's copies do not wait for this step's kernels),
    # the prefill of row b starts when its three inputs have arrived, and its output goes back on a third stream.
    h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    row_caches = [attention.FBLACache(cache.coarse[b:b + 1], cache.fine[b:b + 1], cache.meta[b:b + 1], cache.sink_k[b:b + 1], cache.sink_v[b:b + 1],
                                      cache.open_k[b:b + 1], cache.open_v[b:b + 1], 0, S, cache.format) for b in range(nb)]
    sets = [tuple(torch.empty_like(x) for x in (qd, kd, vd)) for _ in range(2)]
    set_free = [None, None]  # the event after which a set's buffers may be overwritten

    def step_e2e(i):
        dq, dk, dv = sets[i & 1]
        ready = []
        with torch.cuda.stream(h2d):
            if set_free[i & 1] is not None:
                h2d.wait_event(set_free[i & 1])
            for b in range(nb):
                dq[b:b + 1].copy_(host[0][b:b + 1], non_blocking=True)
                dk[b:b + 1].copy_(host[1][b:b + 1], non_blocking=True)
                dv[b:b + 1].copy_(host[2][b:b + 1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(h2d)
                ready.append(ev)
        for b in range(nb):
            main.wait_event(ready[b])
            row_caches[b].tokens = 0
            o = attention.prefill(dq[b:b + 1], dk[b:b + 1], dv[b:b + 1], row_caches[b])
            done = torch.cuda.Event()
            done.record(main)
            o.record_stream(d2h)
            with torch.cuda.stream(d2h):
                d2h.wait_event(done)
                out_host[b:b + 1].copy_(o, non_blocking=True)
        set_free[i & 1] = torch.cuda.Event()
        set_free[i & 1].record(main)

    ms_e2e, _, _ = timed_blocks(D, step_e2e, steps, 3)
    flops = 4.0 * 128 * B * QH * S * (S + 1) / 2
    p = peaks()
    peak, peak_kind = (p["bf16_tflops_sustained"], "measured, sustained") if "bf16_tflops_sustained" in p else (1400.0, "fallback")
    ach = flops / (ms * 1e-3) / 1e12
    return dict(metric="prefill_tflops", value=ach, unit="TFLOP/s", ms_per_step=ms, blocks=blocks,
                config=dict(workload=cfg["name"], l2="q + k + v + cache per step exceed L2", batch=B, q_heads=QH, kv_heads=KH, tokens=S, mode=mode,
                            sharding=("(batch row, KV head) units over %d GPUs, no exchange" % world) if D.world > 1 else "one GPU"),
                e2e=dict(value=flops / (ms_e2e * 1e-3) / 1e12, unit="TFLOP/s", h2d_bytes_per_step=sum(x.numel() * 2 for x in host) * world,
                         d2h_bytes_per_step=out_host.numel() * 2 * world),
                roofline=dict(bound="tensor", achieved=ach, peak=peak * world, unit="TFLOP/s", frac=ach / (peak * world), traffic=None, peak_kind=peak_kind,
                              kernel="attend_tc_kernel (more than 95 % of the prefill call: close, attention, finish)", algorithmic_flops=flops,
                              operands="FP16 products of 6-bit codes and int8 queries, FP32 accumulation in tensor memory"),
                dtype="f16 x f16 -> f32", tokens_per_s=B * S / (ms * 1e-3))


# ---- sequence split (configs[2]) ----------------------------------------------------------------------------------------------
def run_seqsplit(D, cfg, args):
    """One sequence (batch 1, 32q/8kv, 3+3, plain N(0,1)) split over the ranks by whole groups; every decode step = two
    local passes + two small exchanges (row masses, partial sums)."""
    import torch
    import torch.distributed as dist
    from mlops_b200.attention import sharded
    from tests import datagen

    tokens = cfg["tokens"]
    plan = sharded.plan_shards(tokens, D.world)[D.rank]
    n = plan.token_end - plan.token_first + plan.extra
    q, _, _ = datagen.baseline_case(1003, 1, 32, 8, 1, outliers=False)
    qd = bf16(q).to(D.dev)
    chunks_k, chunks_v = [], []
    for c0 in range(0, n, 65536):  # the rank's tokens, generated in chunks to bound host memory
        _, k, v = datagen.baseline_case(1003 + 977 * D.rank + c0, 1, 32, 8, min(65536, n - c0), outliers=False)
        chunks_k.append(bf16(k).to(D.dev)); chunks_v.append(bf16(v).to(D.dev))
    shard = sharded.encode_shard(torch.cat(chunks_k, 2), torch.cat(chunks_v, 2), "3+3", plan)
    del chunks_k, chunks_v
    group = dist.group.WORLD if D.world > 1 else None
    for _ in range(3):
        sharded.decode(qd, shard, group)
    torch.cuda.synchronize()
    # The whole step as ONE CUDA graph: the two exchanges are peer stores and bounded polls inside the step's own kernels
    # (mlops_fbla_shard_step). If the peer-mapped mailboxes cannot be set up: the local segments as graphs around two
    # eager NCCL exchanges.
    runner, launch = None, "eager launches, NCCL exchanges"
    try:
        runner = sharded.LinkedDecode(qd, shard, group)
        runner()
        torch.cuda.synchronize()
        if runner.status() != 0:
            raise RuntimeError(f"link status {runner.status()}")
        launch = "one CUDA graph; exchanges by peer stores and bounded polls (no NCCL on the path)"
    except Exception as exc:  # noqa: BLE001
        print(f"linked step unavailable ({type(exc).__name__}: {exc}); falling back to NCCL exchanges", file=sys.stderr)
        runner = None
        try:
            runner = sharded.GraphedDecode(qd, shard, group)
            runner()
            torch.cuda.synchronize()
            launch = "cuda graphs around eager NCCL exchanges"
        except Exception as exc2:  # noqa: BLE001
            runner = None
            print(f"graph capture unavailable ({type(exc2).__name__}: {exc2}); timing eager launches", file=sys.stderr)

    def step(i):
        if runner is not None:
            runner()
        else:
            sharded.decode(qd, shard, group)

    ms, blocks, clocks = timed_blocks(D, step, args.steps, args.warmup)
    groups = tokens // 128
    coarse = 8 * ((groups - 2) * (8 * 1536 + 1024) + (128 + 128) * 512)
    peak, peak_kind = hbm_peak()
    ach = coarse / (ms * 1e-3) / 1e9
    return dict(metric=METRIC, value=1000.0 / ms, unit=UNIT, ms_per_step=ms, blocks=blocks,
                config=dict(workload=cfg["name"], tokens=tokens, l2="cache larger than L2", launch=launch,
                            sharding="the sequence's groups over %d GPUs; two exchanges per step (4 B and 528 B per row and rank)" % D.world),
                roofline=dict(bound="hbm", achieved=ach, peak=peak * D.world, unit="GB/s", frac=ach / (peak * D.world), traffic=None, peak_kind=peak_kind,
                              algorithmic_bytes=coarse, note="coarse planes + metadata + BF16 windows only (refined share not counted)"),
                dtype="u8")


# ---- CPU legs ---------------------------------------------------------------------------------------------------------------------
def cpu_baseline(cfg, seconds=12.0):
    """The oracle's port of the reference's host-side float64 decode model on the workload's own inputs (cache prebuilt by the
    oracle's quantizer, not timed), repeated for about `seconds`."""
    from oracle import fbla_oracle as orc
    from tests import datagen
    orc.set_threads(os.cpu_count() or 1)
    q, k, v = datagen.baseline_case(cfg["seed"], cfg["batch"], cfg["q_heads"], cfg["kv_heads"], cfg["tokens"], outliers=cfg["outliers"])
    cache = orc.encode(k, v, cfg["mode"])
    times = []
    t_end = time.perf_counter() + seconds
    while not times or (time.perf_counter() < t_end and len(times) < 20):
        t0 = time.perf_counter()
        orc.decode(q, cache)
        times.append(time.perf_counter() - t0)
    dt = float(np.median(times))
    cores = min(orc.threads(), cfg["batch"] * cfg["kv_heads"])  # the model runs one thread per (batch row, KV head)
    return dict(value=cfg["batch"] / dt, unit=UNIT, cores=cores, kind="port",
                sample=f"the whole workload ({cfg['batch']} x {cfg['q_heads']} rows over {cfg['tokens']} tokens) x {len(times)} decodes of the float64 model on "
                       f"the packed cache, {sum(times):.1f} s, median taken; {orc.threads()} threads available, {cores} usable")


def run_reference(args):
    """The reference arm: the reference's host-side path (the oracle port of its float64 model) on this machine's cores."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cfg = WORKLOADS[args.workload if WORKLOADS[args.workload]["kind"] == "decode" else "decode_128k"]
    base = cpu_baseline(cfg, seconds=min(60.0, 6.0 * max(1, args.steps)))
    v = base["value"]
    line = dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=1000.0 * cfg["batch"] / v,
                higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f64", data="synthetic", impl="reference",
                config=dict(workload=cfg["name"], **{k: cfg[k] for k in ("batch", "q_heads", "kv_heads", "tokens", "mode")}),
                cpu_baseline=base, e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))


# ---- driver -------------------------------------------------------------------------------------------------------------------------
def run_workload(D, name, args, headline):
    cfg = dict(WORKLOADS[name], key=name)
    if cfg["kind"] == "decode":
        rec = run_decode(D, cfg, args, headline)
        return None if rec is None else (decode_record(cfg, rec, D.world), rec)
    if cfg["kind"] == "serving":
        return run_serving(D, cfg, args), None
    if cfg["kind"] == "prefill":
        return run_prefill(D, cfg, args), None
    return run_seqsplit(D, cfg, args), None


def main():
    global MIN_TIMED_S
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50, help="steps per timed block (blocks repeat until 0.5 s has been timed)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_128k", choices=sorted(WORKLOADS),
                    help="the line's workload; the default also measures the other configurations as sub-records")
    ap.add_argument("--no-subs", action="store_true", help="measure the named workload only (short runs under a profiler)")
    ap.add_argument("--min-time", type=float, default=MIN_TIMED_S,
                    help="seconds to time at least, in blocks of --steps steps (0: one block; for captures under a profiler)")
    args = ap.parse_args()
    MIN_TIMED_S = args.min_time
    if args.impl == "reference":
        return run_reference(args)
    import torch
    D = Dist()
    res = run_workload(D, args.workload, args, True)
    subs = {}
    if args.workload == "decode_128k" and not args.no_subs:
        names = SUBS + (["seqsplit_256k"] if D.world > 1 else [])
        for name in names:
            torch.cuda.empty_cache()
            r = run_workload(D, name, args, False)
            if r is not None:
                subs[name] = r[0]
    if D.rank == 0 and res is not None:
        line, rec = res
        kind = WORKLOADS[args.workload]["kind"]
        launches = {"decode": 4, "serving": 4, "prefill": 3, "seqsplit": 9}[kind]
        out = dict(metric=line["metric"], value=line["value"], unit=line["unit"], n_gpus=D.world, steps=args.steps, warmup=max(args.warmup, 3),
                   ms_per_step=line["ms_per_step"], blocks=line["blocks"], higher_is_better=True, scaling="strong", vs_baseline=None,
                   dtype=line["dtype"], data="synthetic", config=line["config"], e2e=line.get("e2e"),
                   gpu_launches=launches * args.steps * line["blocks"], roofline=line["roofline"],
                   clocks=(rec or {}).get("clocks") if rec else None)
        if "ref_gpu" in line:
            out["ref_gpu"] = line["ref_gpu"]
        if D.world == 1 and kind == "decode" and not args.no_subs:
            out["cpu_baseline"] = cpu_baseline(WORKLOADS[args.workload])
        if subs:
            out["sub"] = subs
        print(json.dumps(out))
    D.close()


if __name__ == "__main__":
    main()
