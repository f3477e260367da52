"""Headline benchmark of the FBLA hot path: batched compressed-KV decode.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): BASELINE configs[1] -- batch 8, 32 query heads / 8 KV heads, head_dim 128, context 16384 per
sequence (131072 context tokens in all), 4+2 mode, seeded BF16 N(0,1) inputs with 4 outlier channels per KV head
scaled x8, softmax scale 1/sqrt(128), default tau. One step = one decode call (one new token per sequence) over the
resident compressed cache, which the library itself wrote (quantize-on-write).
N > 1: one process per GPU (torchrun), each rank decodes its own batch of 8 sequences -- the path shards by batch row
and KV head with no exchange -- so per-GPU work is fixed ("weak") and value = tokens of all ranks / max time.

Prints ONE JSON line: metric decode tokens/s with the cache resident in HBM (`value`), the same through the Python
interface with host q / output buffers (`e2e`), the roofline of the dominant kernel, a CPU baseline (the oracle's port
of the reference's host-side model, a bounded sample), clocks sampled during the timed region.
`--impl reference` times the reference's host-side path on the CPU cores of this machine (the oracle port).
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

CFG = dict(batch=8, q_heads=32, kv_heads=8, tokens=16384, mode="4+2", seed=1002, outliers=True,
           name="decode B8 32q/8kv ctx16384 4+2 (BASELINE configs[1])")
# the metric's headline shape: one sequence of 131 072 tokens, plain N(0,1) inputs as in configs[2]
LONG = dict(batch=1, q_heads=32, kv_heads=8, tokens=131072, seed=1003, outliers=False)
METRIC, UNIT = "decode_tokens_per_s", "tokens/s"
# dram__bytes_read.sum + dram__bytes_write.sum of the four kernels of one decode step of this workload, from the ncu capture of
# `bench.py --steps 4 --warmup 3` summarised in profiles/decode_b8_ctx16k_4p2_launches.md (coarse 153.7 MB, select 1.7 MB,
# refine 164.7 MB, merge 6.5 MB); reported only while the refined share is the one of that capture
NCU_DRAM_BYTES_PER_STEP = 326601984


def make_inputs(rank=0):
    from tests import datagen
    return datagen.baseline_case(CFG["seed"] + 7919 * rank, CFG["batch"], CFG["q_heads"], CFG["kv_heads"], CFG["tokens"], outliers=CFG["outliers"])


def algorithmic_bytes(share):
    """Bytes one decode must move (the reference bench's accounting, attention/fbla/bench/bench_fbla.cu:136-141):
    coarse records + 1 KiB metadata of every closed group, the BF16 sink and open tokens (K and V), and coarse + fine
    records of the share of closed sub-blocks that some query of the KV head refines."""
    cb, fb = (3, 3) if CFG["mode"] == "3+3" else (4, 2)
    heads = CFG["batch"] * CFG["kv_heads"]
    groups = (CFG["tokens"] + 127) // 128
    closed = max(groups - 2, 0)
    open_tokens = CFG["tokens"] - 128 * (groups - 1)
    rc, rf = 2 * cb * 256, 2 * fb * 256
    coarse = heads * closed * (8 * rc + 1024)
    windows = heads * (128 + open_tokens) * 128 * 2 * 2
    refine = share * heads * closed * 8 * (rc + rf)
    return coarse + windows + refine, dict(coarse_and_meta=coarse, bf16_windows=windows, refine=refine)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

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


def cpu_baseline(rows=8, repeats=3):
    """The oracle's port of the reference's host-side decode model on `rows` of the workload's batch rows, `repeats` times."""
    from oracle import fbla_oracle as orc
    from tests import datagen
    rows = min(rows, CFG["batch"])
    q, k, v = datagen.baseline_case(CFG["seed"], rows, CFG["q_heads"], CFG["kv_heads"], CFG["tokens"], outliers=CFG["outliers"])
    cache = orc.encode(k, v, CFG["mode"])
    t0 = time.perf_counter()
    for _ in range(repeats):
        _, stats = orc.decode(q, cache, stats=True)
    dt = time.perf_counter() - t0
    return dict(value=rows * repeats / dt, unit=UNIT, cores=orc.threads(), kind="port",
                sample=f"{rows} of {CFG['batch']} batch rows of the workload x {repeats} (float64 decode model on the packed cache, cache prebuilt), {dt:.1f} s"), stats


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_baseline(8, 1)
    base = None
    for _ in range(max(1, min(args.steps, 3))):
        base, _ = cpu_baseline(8, 2)
        vals.append(base["value"])
    v = float(np.median(vals))
    base["value"] = v
    line = dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=len(vals), warmup=1, ms_per_step=1000.0 * CFG["batch"] / v,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f64", data="synthetic", impl="reference",
                config=dict(workload=CFG["name"], **{k: CFG[k] for k in ("batch", "q_heads", "kv_heads", "tokens", "mode")}),
                cpu_baseline=base, e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))


def run_ours(args):
    import ctypes

    import torch
    import torch.distributed as dist

    from mlops_b200 import attention
    from mlops_b200.attention import _C

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    q, k, v = make_inputs(rank)
    bf = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)
    q_host = bf(q).pin_memory()
    qd = q_host.to(dev)
    # two caches (the same tokens, separate memory), alternated step by step: the working set (2 x 210 MB) exceeds L2
    copies = []
    kd, vd = bf(k).to(dev), bf(v).to(dev)
    for _ in range(2):
        copies.append(attention.encode(kd, vd, CFG["mode"]))
    del kd, vd
    c0 = copies[0]
    cfg = _C.Config(CFG["batch"], CFG["q_heads"], CFG["kv_heads"], c0.tokens, 0.0, 0.0, c0.format, c0.capacity, 0, 0, 0, 0, 0)
    nbytes = _C.lib.mlops_fbla_decode_scratch_bytes(ctypes.byref(cfg))
    scratch = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=dev)
    out = torch.empty_like(qd)
    caches = [_C.Cache(c.coarse.data_ptr(), c.fine.data_ptr(), c.meta.data_ptr(), c.sink_k.data_ptr(), c.sink_v.data_ptr(), c.open_k.data_ptr(),
                       c.open_v.data_ptr(), None) for c in copies]

    def step(i, stream):
        st = _C.lib.mlops_fbla_decode(ctypes.byref(cfg), qd.data_ptr(), ctypes.byref(caches[i & 1]), out.data_ptr(), scratch.data_ptr(), nbytes,
                                      ctypes.c_void_p(stream.cuda_stream))
        if st:
            raise RuntimeError(_C.last_error())

    stream = torch.cuda.current_stream()
    for i in range(max(args.warmup, 3)):
        step(i, stream)
    torch.cuda.synchronize()
    status = scratch[-256:].view(torch.int32)[:2].tolist()
    if status[0]:
        raise RuntimeError(f"a bounded wait gave up: status {status}")
    # refined share of (KV head, sub-block) pairs, from the device's own select pass
    vheads, nsl = CFG["batch"] * CFG["kv_heads"], max(1, ((CFG["tokens"] + 127) // 128 * 8 + 1023) // 1024)
    share = refine_share(scratch, cfg, _C, vheads, nsl)
    abytes, parts = algorithmic_bytes(share)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: K steps between CUDA events on the launching stream ----------------------------
    sampler = ClockSampler(local)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    ev0.record(stream)
    for i in range(args.steps):
        step(i, stream)
    ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.result()
    # ---- end to end through the Python interface: host q -> device, decode, output -> host, every step -----------------
    light = os.environ.get("FBLA_BENCH_LIGHT") == "1"  # profiling runs: skip the end-to-end and CPU legs
    out_host = torch.empty(q_host.shape, dtype=torch.bfloat16).pin_memory()
    for i in range(3):
        attention.decode(q_host.to(dev, non_blocking=True), copies[i & 1])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(1 if light else args.steps):
        o = attention.decode(q_host.to(dev, non_blocking=True), copies[i & 1])
        out_host.copy_(o, non_blocking=True)
    e1.record(stream)
    barrier()
    ms_e2e = e0.elapsed_time(e1) * (args.steps if light else 1)
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak, peak_kind = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
        per_step = ms / args.steps
        achieved = abytes / (per_step * 1e-3) / 1e9
        value = world * CFG["batch"] / (per_step * 1e-3)
        line = dict(metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=per_step,
                    higher_is_better=True, scaling="weak", vs_baseline=None, dtype="u8", data="synthetic",
                    config=dict(workload=CFG["name"] + "; per rank", l2="two cache copies alternated, together larger than L2",
                                refined_share=share, **{k: CFG[k] for k in ("batch", "q_heads", "kv_heads", "tokens", "mode")}),
                    e2e=dict(value=world * CFG["batch"] / (ms_e2e / args.steps * 1e-3), unit=UNIT, h2d_bytes_per_step=q_host.numel() * 2,
                             d2h_bytes_per_step=out_host.numel() * 2),
                    gpu_launches=4 * args.steps,
                    roofline=dict(bound="hbm", achieved=achieved, peak=peak, unit="GB/s", frac=achieved / peak,
                                  traffic=NCU_DRAM_BYTES_PER_STEP if CFG["tokens"] == 16384 and abs(share - 0.776) < 0.01 else None, peak_kind=peak_kind,
                                  kernel="decode call (coarse + select + refine + merge)", algorithmic_bytes=abytes, bytes_parts=parts),
                    clocks=clocks)
        if world == 1 and not light:
            base, stats = cpu_baseline(8, 3)
            line["cpu_baseline"] = base
            line["config"]["oracle_refined_share"] = stats[3] / max(1, stats[2])
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def refine_share(scratch, cfg, _C, vheads, nsl):
    """Fraction of closed (KV head, sub-block) pairs the select pass listed: total items / closed sub-blocks. The total is
    the last word of the item_off array (offsets follow the scratch layout of mlops_b200/csrc/host/fbla_api.cpp)."""
    import torch
    up = lambda n: (n + 255) & ~255
    items_total_off = scratch.numel() - 256 - up((vheads + 1) * 4) + vheads * 4
    total = int(scratch[items_total_off:items_total_off + 4].view(torch.int32).item())
    groups = (cfg.tokens + 127) // 128
    closed_blocks = vheads * max(groups - 2, 0) * 8
    return total / max(1, closed_blocks)


def run_seqsplit(args):
    """BASELINE configs[2]: one sequence (batch 1, 32q/8kv, 3+3, plain N(0,1)) of 256K or 1M tokens split over the
    ranks by whole groups; every decode step = two local passes + two NCCL exchanges (mass, partial sums)."""
    import torch
    import torch.distributed as dist

    from mlops_b200.attention import sharded
    from tests import datagen

    tokens = 262144 if args.workload == "seqsplit_256k" else 1 << 20
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    plan = sharded.plan_shards(tokens, world)[rank]
    n = plan.token_end - plan.token_first + plan.extra
    bf = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)
    q, _, _ = datagen.baseline_case(1003, 1, 32, 8, 1, outliers=False)
    qd = bf(q).to(dev)
    chunks_k, chunks_v = [], []
    for c0 in range(0, n, 65536):  # the rank's tokens, generated in chunks to bound host memory
        _, k, v = datagen.baseline_case(1003 + 977 * rank + c0, 1, 32, 8, min(65536, n - c0), outliers=False)
        chunks_k.append(bf(k).to(dev)); chunks_v.append(bf(v).to(dev))
    shard = sharded.encode_shard(torch.cat(chunks_k, 2), torch.cat(chunks_v, 2), "3+3", plan)
    del chunks_k, chunks_v
    group = dist.group.WORLD if world > 1 else None
    for _ in range(max(args.warmup, 3)):
        out = sharded.decode(qd, shard, group)
    torch.cuda.synchronize()
    # the step's local segments as CUDA graphs, the two exchanges as ordinary NCCL calls between them: the step is a
    # handful of ~30 us kernels, so host launch overhead would otherwise be what is measured
    graph, mode_ = None, "eager"
    try:
        graph = sharded.GraphedDecode(qd, shard, group)
        out = graph()
        torch.cuda.synchronize()
        mode_ = "cuda graphs around eager exchanges" if world > 1 else "cuda graphs"
    except Exception as exc:  # noqa: BLE001
        graph = None
        print(f"graph capture unavailable ({type(exc).__name__}: {exc}); timing eager launches", file=sys.stderr)
    if world > 1:
        dist.barrier()
    stream = torch.cuda.current_stream()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    sampler.start()
    ev0.record(stream)
    for _ in range(args.steps):
        if graph is not None:
            out = graph()
        else:
            out = sharded.decode(qd, shard, group)
    ev1.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / args.steps
    clocks = sampler.result()
    if rank == 0:
        groups = tokens // 128
        coarse = 8 * ((groups - 2) * (8 * 1536 + 1024) + (128 + 128) * 512)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = peaks.get("hbm_gbs", 6650.0)
        ach = coarse / (ms * 1e-3) / 1e9
        print(json.dumps(dict(metric=METRIC, value=1000.0 / ms, unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3), ms_per_step=ms,
                              higher_is_better=True, scaling="strong", vs_baseline=None, dtype="u8", data="synthetic",
                              config=dict(workload=f"sequence-split decode B1 32q/8kv ctx{tokens} 3+3 (BASELINE configs[2])", tokens=tokens, l2="cache larger than L2", launch=mode_),
                              gpu_launches=(2 + 3 + 2) * args.steps,
                              roofline=dict(bound="hbm", achieved=ach, peak=peak * world, unit="GB/s", frac=ach / (peak * world), traffic=None,
                                            algorithmic_bytes=coarse, note="coarse planes + metadata + BF16 windows only (refined share not counted)"),
                              clocks=clocks)))
    if world > 1:
        dist.destroy_process_group()


def run_prefill(args):
    """BASELINE configs[3]: causal prefill, batch 4, sequence 8192, 32q/8kv, 4+2. One step = one prefill call on an empty
    cache: quantize-on-write of the chunk's groups, attention over the compressed cache (tensor cores), window update.
    N > 1: every rank prefills its own batch (weak). FLOPs: 4 * 128 per (query, attended key) pair (QK and PV)."""
    import torch
    import torch.distributed as dist

    from mlops_b200 import attention
    from tests import datagen

    B, QH, KH, S, mode = (4 if args.workload == "prefill_b4" else 1), 32, 8, 8192, "4+2"  # prefill_b1: the small case for profiler captures
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    q, k, v = datagen.baseline_case(1004 + 7919 * rank, B, QH, KH, S, q_rows=S, outliers=True)
    bf = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)
    host = [bf(x).pin_memory() for x in (q, k, v)]
    qd, kd, vd = [x.to(dev) for x in host]
    cache = attention.empty(B, KH, S, mode, device=dev)
    steps, warmup = min(args.steps, 20), max(min(args.warmup, 5), 3)

    def step():
        cache.tokens = 0  # the same buffers, refilled from the start
        return attention.prefill(qd, kd, vd, cache)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        out = step()
    stream = torch.cuda.current_stream()
    sampler = ClockSampler(local)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    ev0.record(stream)
    for _ in range(steps):
        out = step()
    ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1) / steps
    clocks = sampler.result()
    out_host = torch.empty(out.shape, dtype=torch.bfloat16).pin_memory()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(steps):
        cache.tokens = 0
        o = attention.prefill(host[0].to(dev, non_blocking=True), host[1].to(dev, non_blocking=True), host[2].to(dev, non_blocking=True), cache)
        out_host.copy_(o, non_blocking=True)
    e1.record(stream)
    barrier()
    ms_e2e = e0.elapsed_time(e1) / steps
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = t.tolist()
    if rank == 0:
        flops = 4.0 * 128 * B * QH * S * (S + 1) / 2
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak, peak_kind = (peaks["bf16_tflops_sustained"], "measured, sustained") if "bf16_tflops_sustained" in peaks else (1400.0, "fallback")
        ach = flops / (ms * 1e-3) / 1e12
        rows_per_cta = 256
        print(json.dumps(dict(metric="prefill_tflops", value=world * ach, unit="TFLOP/s", n_gpus=world, steps=steps, warmup=warmup, ms_per_step=ms,
                              higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f16 products of 6-bit codes and int8 queries, f32 accumulation",
                              data="synthetic",
                              config=dict(workload=f"causal prefill B{B} S8192 32q/8kv 4+2 (BASELINE configs[3]" + ("" if B == 4 else ", one of its four sequences") + "); per rank", l2="q + k + v + cache = 0.5 GB per step > L2",
                                          batch=B, q_heads=QH, kv_heads=KH, tokens=S, mode=mode),
                              e2e=dict(value=world * flops / (ms_e2e * 1e-3) / 1e12, unit="TFLOP/s", h2d_bytes_per_step=sum(x.numel() * 2 for x in host),
                                       d2h_bytes_per_step=out_host.numel() * 2),
                              gpu_launches=3 * steps,
                              roofline=dict(bound="tensor", achieved=ach, peak=peak, unit="TFLOP/s", frac=ach / peak, traffic=None, peak_kind=peak_kind,
                                            kernel="prefill call (close + attend_tc + finish); attend_tc is > 95 % of it", algorithmic_flops=flops,
                                            rows_per_cta=rows_per_cta),
                              clocks=clocks)))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_b8", choices=["decode_b8", "decode_128k_3p3", "decode_128k_4p2", "seqsplit_256k", "seqsplit_1m", "prefill_b4", "prefill_b1"],
                    help="decode_b8: the headline (BASELINE configs[1]); decode_128k_*: one 131 072-token sequence; seqsplit_*: one long sequence split over the ranks (configs[2]); "
                         "prefill_b4: causal prefill in TFLOP/s (configs[3]); prefill_b1: one of its four sequences (profiler captures)")
    args = ap.parse_args()
    if args.workload.startswith("decode_128k"):  # the metric's headline context length, batch 1, either format
        mode = "3+3" if args.workload.endswith("3p3") else "4+2"
        CFG.update(LONG, mode=mode, name=f"decode B1 32q/8kv ctx131072 {mode} (the metric's headline context)")
        args.workload = "decode_b8"
    if args.workload.startswith("prefill") and args.impl == "ours":
        return run_prefill(args)
    if args.workload != "decode_b8" and args.impl == "ours":
        return run_seqsplit(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
