"""Benchmark of the paged-KV decode step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5a|c5b] [--impl reference]

One step = the hot path on one batch: append one token per sequence into its page, then
single-query attention over the whole cache through the block table.  Prints ONE JSON line.

* ``value``     decode tokens/s, whole job, inputs resident in HBM (CUDA events, max over ranks).
* ``e2e``       the same step driven from pinned HOST buffers: q / new K,V / slot mapping / lengths
                copied in, result copied out, every step.
* ``roofline``  algorithmic bytes of the attention call / its mean duration, against the measured
                HBM copy bandwidth of this pool's B200s.
* ``cpu_baseline``  the CPU checker (the reference's torch path restated) on a bounded sample.

With ``--gpus N`` (under torchrun) every rank runs the same per-GPU workload on its own page pool
with no collective on the data path ("weak" scaling); ``--workload c5b`` is the head-parallel form
of one long sequence with an NCCL all-gather of the outputs.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import iva_b200  # noqa: E402
from iva_b200 import workloads  # noqa: E402

METRIC = "paged decode-attn GB/s (% of HBM peak) and decode tok/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch from an ncu capture,
# as a multiple of the algorithmic bytes of that launch (see profiles/); None until captured.
# c2: 8-sequence case, 539.10 MB read + 4.80 MB written for 537.14 MB algorithmic;
# c3: 32-sequence case, 350.44 MB + 7.68 MB for 349.93 MB.  Traffic grows with the tokens read, so the
# ratio carries over to the full-size launch.
NCU_TRAFFIC_RATIO = {"c2": (539.10 + 4.80) / 537.14, "c3": (350.44 + 7.68) / 349.93, "c5a": (350.44 + 7.68) / 349.93}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---- algorithmic bytes (minimum traffic: every K/V element once, q/out/lse/tables once) ------------

def attention_bytes(wl, lens):
    elt = wl.k_pool.element_size()
    tokens = int(lens.sum())
    pages = int(((lens + wl.page_size - 1) // wl.page_size).sum())
    B = wl.batch
    return (2 * tokens * wl.n_kv_heads * wl.head_dim * elt + 2 * B * wl.n_q_heads * wl.head_dim * elt
            + B * wl.n_q_heads * 4 + pages * 4 + B * 4)


def append_bytes(wl):
    elt = wl.k_pool.element_size()
    T = wl.k_new.shape[0]
    return 4 * T * wl.n_kv_heads * wl.head_dim * elt + T * 8


def gather_bytes(wl, lens):
    elt = wl.k_pool.element_size()
    tokens = int(lens.sum())
    pages = int(((lens + wl.page_size - 1) // wl.page_size).sum())
    return 2 * (2 * tokens * wl.n_kv_heads * wl.head_dim * elt) + 2 * pages * 4


# ---- clocks ----------------------------------------------------------------------------------------

class ClockSampler:
    """Samples nvidia-smi while the timed region runs (reads only; never changes a setting)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw,clocks.mem")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        def num(x):
            try:
                return float(x)
            except ValueError:
                return None
        power = [num(r[6]) for r in self.rows if len(r) > 6 and num(r[6]) is not None]
        mem = [num(r[7]) for r in self.rows if len(r) > 7 and num(r[7]) is not None]
        return {"sm_mhz": statistics.median(int(r[0]) for r in self.rows), "sm_min_mhz": min(int(r[0]) for r in self.rows),
                "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons, "samples": len(self.rows),
                "power_w_max": max(power) if power else None, "mem_mhz": statistics.median(mem) if mem else None}


# ---- workloads ---------------------------------------------------------------------------------------

def build_workload(name, device, rank, world, args):
    if name == "c2":
        return workloads.config_c2(device=device, seed=rank, batch=args.batch or 64, context=args.context or 4096)
    if name == "c3":
        return workloads.config_c3(device=device, seed=rank, batch=args.batch or 128)
    if name == "c4":
        return workloads.config_c4(device=device, seed=rank, n_seq=args.batch or 256)
    if name == "c5a":
        return workloads.config_c5a(device=device, n_seq=args.batch or 1024, context=args.context or 8192,
                                    rank=rank, world=world)
    if name == "c5b":
        return workloads.config_c5b(device=device, context=args.context or 131072)
    raise SystemExit(f"unknown workload {name}")


WORKLOAD_TEXT = {"c2": "1xB200 MHA decode step (append 1 token/seq + paged attention)",
                 "c3": "1xB200 GQA decode step, ragged log-normal contexts",
                 "c4": "append/gather stress (512-token fp16 chunks, then gather all)",
                 "c5a": "request-sharded GQA decode, 1024 seq x 8192 split over ranks",
                 "c5b": "one 131072-token sequence, KV heads split over ranks + all-gather"}


def workload_shape(name, args, rank, world):
    """Lengths and head layout of a workload without building its pools (the reference arm reports
    the GPU arm's config although it only times a sample of it)."""
    if name == "c2":
        ctx, hq, hkv, dt, new, free = torch.full((args.batch or 64,), args.context or 4096), 32, 32, "bfloat16", 1, 0.0
    elif name == "c3":
        ctx, hq, hkv, dt, new, free = workloads.ragged_lengths(args.batch or 128, rank), 32, 8, "bfloat16", 1, 0.10
    elif name == "c4":
        g = torch.Generator().manual_seed(rank)
        ctx, hq, hkv, dt, new, free = torch.randint(0, 8193, (args.batch or 256,), generator=g), 32, 32, "float16", 512, 0.0
    elif name == "c5a":
        ctx, hq, hkv, dt, new, free = torch.full(((args.batch or 1024) // world,), args.context or 8192), 32, 8, "bfloat16", 1, 0.0
    else:
        ctx, hq, hkv, dt, new, free = torch.full((1,), args.context or 131072), 32, 8, "bfloat16", 1, 0.0
    pages = int(((ctx + new + 15) // 16).sum())
    return {"ctx": ctx, "hq": hq, "hkv": hkv, "dtype": dt, "pool_pages": int(-(-pages * (1.0 + free) // 1))}


def describe(name, args, rank, world, kv_fp8=False):
    sh = workload_shape(name, args, rank, world)
    ctx, elt = sh["ctx"], (1 if kv_fp8 else 2)
    kv_bytes = 2 * int((ctx + 1).sum()) * sh["hkv"] * 128 * elt
    return {
        "workload": WORKLOAD_TEXT[name], "name": name, "batch_per_gpu": int(ctx.numel()), "q_heads": sh["hq"],
        "kv_heads": sh["hkv"], "head_dim": 128, "page_size": 16,
        "kv_dtype": "float8_e4m3fn" if kv_fp8 else sh["dtype"],
        "context_min": int(ctx.min()), "context_max": int(ctx.max()), "context_sum": int(ctx.sum()),
        "pool_pages": sh["pool_pages"],
        "parallelism": "1 GPU" if world == 1 else f"{world} GPUs, one process each",
        "l2": "K/V read per step exceed the 126 MB L2 and are not reused between steps"
              if kv_bytes > 4 * 126e6 else "L2 flushed between timed steps",
    }


def live_copy_bandwidth(dev):
    """STREAM-style copy on THIS GPU, the way the recorded peak was taken (b.copy_(a) over 1 Gi bf16
    elements, read+write bytes, best of 10): B200s of one pool differ by a few per cent, so the
    live figure is reported next to the recorded one."""
    n = 1 << 30
    a = torch.empty(n, dtype=torch.bfloat16, device=dev)
    b = torch.empty(n, dtype=torch.bfloat16, device=dev)
    a.fill_(1)
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        b.copy_(a)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    del a, b
    torch.cuda.empty_cache()
    return 2 * n * 2 / (best * 1e-3) / 1e9


# ---- the GPU arm --------------------------------------------------------------------------------------

def time_region(fn, steps, flush=None):
    """CUDA-event time of ``steps`` calls on the current stream, in ms (sum of per-call events so
    that an optional L2 flush between calls stays outside the measurement)."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        if flush is not None:
            flush()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


def run_gpu(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    lib = iva_b200.load_library()
    name = args.workload
    copy_gbs = live_copy_bandwidth(dev)
    wl = build_workload(name, dev, rank, world, args)
    B = wl.batch
    kv_scales = {}
    if args.kv_fp8:
        if name not in ("c2", "c3", "c5a"):
            raise SystemExit("--kv-fp8 applies to the decode workloads c2, c3, c5a")
        # N(0,1) data: a scale of 1/64 keeps +-7 sigma inside the e4m3 range
        kv_scales = {"k_scale": 1.0 / 64, "v_scale": 1.0 / 64}
        for attr in ("k_pool", "v_pool"):
            pool = getattr(wl, attr)
            q8 = torch.empty(pool.shape, dtype=torch.float8_e4m3fn, device=dev)
            step_rows = 1 << 16
            for lo in range(0, pool.shape[2], step_rows):      # chunked: no full-size fp32 temporary
                q8[:, :, lo:lo + step_rows] = (pool[:, :, lo:lo + step_rows].float() * 64.0).clamp(-448, 448).to(torch.float8_e4m3fn)
            setattr(wl, attr, q8)
        torch.cuda.empty_cache()
    lens = (wl.ctx_len + wl.new_tokens_per_seq).contiguous()
    out = torch.empty(B, wl.n_q_heads, wl.head_dim, device=dev, dtype=wl.dtype) if wl.q is not None else None
    lse = torch.empty(B, wl.n_q_heads, device=dev, dtype=torch.float32) if wl.q is not None else None
    flush_buf = None
    need_flush = wl.q is not None and attention_bytes(wl, lens) <= 4 * 126e6
    if need_flush:
        flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    flush = (lambda: flush_buf.fill_(1)) if need_flush else None

    hp = None
    if name == "c5b":
        from iva_b200.sharding import HeadParallelDecoder
        if world > 1:
            hp = HeadParallelDecoder(wl.n_q_heads, wl.n_kv_heads)
            k_loc, v_loc = hp.local_pools(wl.k_pool, wl.v_pool)
            k_loc, v_loc = k_loc.contiguous(), v_loc.contiguous()      # each rank keeps only its slab
            k_new_loc, v_new_loc = wl.k_new[:, hp.kv_slice].contiguous(), wl.v_new[:, hp.kv_slice].contiguous()
            wl.k_pool, wl.v_pool = k_loc, v_loc                        # drop the full pools
            torch.cuda.empty_cache()

    def append():
        if hp is not None:
            iva_b200.paged_append(k_loc, v_loc, wl.slot_mapping, k_new_loc, v_new_loc, wl.page_size)
        else:
            iva_b200.paged_append(wl.k_pool, wl.v_pool, wl.slot_mapping, wl.k_new, wl.v_new, wl.page_size)

    hp_step = None
    if hp is not None and not args.no_graph:
        hp_step = hp.capture_local(wl.q, k_loc, v_loc, wl.block_table, lens, wl.page_size, wl.scale)

    def attend():
        if hp_step is not None:
            return hp_step()
        if hp is not None:
            return hp.decode(wl.q, k_loc, v_loc, wl.block_table, lens, wl.page_size, wl.scale)
        return iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, wl.page_size,
                                               wl.scale, out=out, lse=lse, **kv_scales)

    gather_offs = None
    if name == "c4":
        gather_offs = torch.zeros(B + 1, dtype=torch.int64, device=dev)
        gather_offs[1:] = torch.cumsum(lens.long(), 0)
        total_tokens = int(gather_offs[-1])

    def gather():
        k = iva_b200.paged_gather(wl.k_pool, wl.block_table, lens, wl.page_size, layout="token_major",
                                  out_offsets=gather_offs, total_tokens=total_tokens)
        v = iva_b200.paged_gather(wl.v_pool, wl.block_table, lens, wl.page_size, layout="token_major",
                                  out_offsets=gather_offs, total_tokens=total_tokens)
        return k, v

    def step():
        append()
        if name == "c4":
            gather()
        else:
            attend()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- device-resident timing (the headline `value`) ----
    launches0 = lib.ivab_launch_count()
    # clocks are sampled from here to the end of the end-to-end leg (a K-step region alone can be
    # shorter than one nvidia-smi sampling period)
    clocks = ClockSampler(local)
    clocks.__enter__()
    barrier()
    per_step = time_region(step, args.steps, flush)
    barrier()
    launches = lib.ivab_launch_count() - launches0
    total_ms = sum(per_step)
    # per-kernel legs, same stream, same conditions
    attn_ms = time_region(attend, args.steps, flush) if name != "c4" else None
    app_ms = time_region(append, args.steps, flush)
    gat_ms = time_region(gather, max(2, args.steps // 4)) if name == "c4" else None
    if dist is not None:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    seqs_total = B * world if name != "c5b" else B
    value = seqs_total * wl.new_tokens_per_seq / (ms_per_step * 1e-3)

    # ---- end to end from pinned host buffers ----
    e2e = None
    if name in ("c2", "c3", "c5a"):
        # the public end-to-end call: inputs in pinned host memory, one CUDA-graph replay per step
        # (H2D of q / new K,V / slot mapping / lengths, append, attention; the kernels store the output
        # straight into the pinned host buffer, d2h_bytes_per_step counts those bytes)
        gs = iva_b200.GraphedDecodeStep(wl.k_pool, wl.v_pool, wl.block_table, wl.n_q_heads, wl.page_size, wl.scale,
                                        token_dtype=wl.dtype, **kv_scales)
        gs.q_host.copy_(wl.q)
        gs.k_new_host.copy_(wl.k_new)
        gs.v_new_host.copy_(wl.v_new)
        gs.slot_mapping_host.copy_(wl.slot_mapping)
        gs.ctx_len_host.copy_(lens)
        torch.cuda.synchronize()

        def e2e_step():
            gs.run()
            return gs.result()                              # the host consumes the result every step

        for _ in range(max(args.warmup, 3)):
            e2e_step()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        a.record(gs.stream)
        for _ in range(args.steps):
            e2e_step()
        b.record(gs.stream)
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = max(a.elapsed_time(b), 0.0)
        if dist is not None:
            t = torch.tensor([e2e_ms, wall_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms, wall_ms = float(t[0].item()), float(t[1].item())
        e2e = {"value": seqs_total / (wall_ms / args.steps * 1e-3), "unit": "decode tok/s",
               "h2d_bytes_per_step": gs.h2d_bytes, "d2h_bytes_per_step": gs.d2h_bytes,
               "ms_per_step": wall_ms / args.steps, "device_ms_per_step": e2e_ms / args.steps,
               "api": "GraphedDecodeStep.run() + result(), host clock around K steps (each step ends in a stream sync)"}
        out.copy_(gs.out_host if gs.direct_host_output else gs._out)

    clocks.__exit__(None, None, None)
    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    if name == "c4":
        dom_bytes, dom_ms, dom_name = gather_bytes(wl, lens), statistics.mean(gat_ms), "paged_gather_kernel (K and V)"
    else:
        wl_local = wl
        dom_bytes = attention_bytes(wl_local, lens) // (world if name == "c5b" else 1)
        dom_ms, dom_name = statistics.mean(attn_ms), "plan_kernel + decode_kernel + merge_kernel (one attention call)"
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    ratio = NCU_TRAFFIC_RATIO.get(name)
    result = {
        "metric": METRIC, "value": value, "unit": "decode tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if name in ("c5a", "c5b") else "weak", "vs_baseline": None,
        "dtype": {"torch.bfloat16": "bf16", "torch.float16": "f16", "torch.float32": "f32"}[str(wl.dtype)],
        "data": "synthetic (seeded N(0,1) K/V/q, shuffled page pool)",
        "config": describe(name, args, rank, world, args.kv_fp8),
        "roofline": {"bound": "hbm", "kernel": dom_name, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                     "algorithmic_bytes": dom_bytes, "ms": dom_ms,
                     "live_copy_GBs_this_gpu": copy_gbs, "frac_of_live_copy": achieved / copy_gbs,
                     "traffic": None if ratio is None else int(dom_bytes * ratio)},
        "kernels": {"append_ms": statistics.mean(app_ms), "append_GBs": append_bytes(wl) / (statistics.mean(app_ms) * 1e-3) / 1e9,
                    "attention_ms": None if attn_ms is None else statistics.mean(attn_ms),
                    "attention_ms_min": None if attn_ms is None else min(attn_ms),
                    "gather_ms": None if gat_ms is None else statistics.mean(gat_ms)},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks.summary(),
    }
    if args.cpu_baseline and world == 1:
        result["cpu_baseline"] = cpu_baseline(name, args, budget_s=12.0)
        result["c1_reference_case"] = c1_case(dev)
    print(json.dumps(result))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ---- the CPU arm (checker timed as a baseline) ------------------------------------------------------------

def cpu_sample(name, args):
    """A bounded sample of the workload: same heads, dtype, page size and context, fewer sequences."""
    if name == "c3":
        return workloads.config_c3(device="cpu", batch=8), "8 of 128 sequences (same length distribution)"
    if name == "c5a":
        return workloads.config_c5a(device="cpu", n_seq=2, context=args.context or 8192), "2 of 1024 sequences"
    if name == "c5b":
        return workloads.config_c5b(device="cpu", context=16384), "one sequence cut to 16384 tokens"
    ctx = args.context or 4096
    return workloads.config_c2(device="cpu", batch=4, context=ctx), f"4 of 64 sequences, context {ctx}, own pool"


def cpu_baseline(name, args, budget_s, kind_label="port"):
    from oracle import paged_ref as ref

    torch.set_num_threads(os.cpu_count() or 1)
    wl, sample = cpu_sample(name if name != "c4" else "c2", args)
    ref.decode_step_ref(wl)                                    # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 200):
        t0 = time.perf_counter()
        ref.decode_step_ref(wl)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": wl.batch / med, "unit": "decode tok/s", "cores": torch.get_num_threads(), "kind": kind_label,
            "sample": f"{sample}; median of {len(times)} steps of the torch-CPU restatement of the reference path "
                      f"(clone+index_copy append, index_select gather, matmul/softmax/matmul)",
            "ms_per_step": med * 1e3,
            "attn_GBs": attention_bytes(wl, wl.ctx_len + 1) / med / 1e9}


def c1_case(dev):
    """The reference's own CPU-runnable configuration run EXACTLY (batch 4, 16 heads, head_dim 64, fp32,
    page 16, contexts U[1,512], 256-page pool, seed 0): one decode step on the host cores (checker)
    and on the GPU (append + attention, CUDA events, L2 flushed between steps)."""
    from oracle import paged_ref as ref

    wl = workloads.config_c1()
    ref.decode_step_ref(wl)
    cpu = []
    for _ in range(20):
        t0 = time.perf_counter()
        ref.decode_step_ref(wl)
        cpu.append(time.perf_counter() - t0)
    d = wl.to(dev)
    lens = (d.ctx_len + 1).contiguous()
    out = torch.empty(wl.batch, wl.n_q_heads, wl.head_dim, device=dev, dtype=wl.dtype)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        iva_b200.paged_append(d.k_pool, d.v_pool, d.slot_mapping, d.k_new, d.v_new, wl.page_size)
        iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, lens, wl.page_size, wl.scale, out=out)

    for _ in range(5):
        step()
    gpu = time_region(step, 50, lambda: flush_buf.fill_(1))
    nbytes = attention_bytes(wl, wl.ctx_len + 1) + append_bytes(wl)
    return {"config": "batch 4, 16 heads, head_dim 64, fp32, contexts " + str(wl.ctx_len.tolist()),
            "cpu_ms_per_step": statistics.median(cpu) * 1e3, "cpu_cores": torch.get_num_threads(),
            "gpu_ms_per_step": statistics.median(gpu), "algorithmic_bytes": nbytes,
            "note": "latency-bound on the GPU: 1 MB of K/V, four kernel launches"}


def run_reference(args):
    """``--impl reference``: the reference's own path on the host cores.  The reference is pure
    Python whose package cannot be imported (syntax errors in three of its modules), so the timed
    code is the checker's restatement of it on PyTorch CPU operators."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload
    base = cpu_baseline(name, args, budget_s=max(5.0, min(60.0, 2.0 * (args.steps + args.warmup))))
    wl, _ = cpu_sample(name if name != "c4" else "c2", args)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "decode tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {"torch.bfloat16": "bf16", "torch.float16": "f16", "torch.float32": "f32"}[str(wl.dtype)],
        "data": "synthetic (seeded N(0,1) K/V/q, shuffled page pool)", "config": describe(name, args, 0, 1),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "decode tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5a", "c5b"])
    ap.add_argument("--batch", type=int, default=0, help="override the number of sequences (small ncu captures)")
    ap.add_argument("--context", type=int, default=0, help="override the context length")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--kv-fp8", action="store_true", help="store K/V as e4m3 with per-tensor scales (c2/c3/c5a)")
    ap.add_argument("--no-graph", action="store_true", help="head-parallel mode: launch eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
