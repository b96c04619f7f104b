"""Benchmark of the paged-KV decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload all|c2|c3|c4|c5a|c5b] [--impl reference]

One step = the hot path on one batch: append one token per sequence into its page, then
single-query attention over the whole cache through the block table.  Prints ONE JSON line.

The headline (``value``, ``e2e``, ``roofline``) is the multi-head decode configuration "c2"
(64 sequences x 32 heads x 4096 keys, bf16), one copy per GPU.  With ``--workload all`` (the
default) the same line carries one sub-record per other configuration:

* ``c3``         ragged grouped-query decode, 128 sequences (1 GPU runs only)
* ``c4``         append / gather stress: 131072 tokens appended, 1.18 M tokens gathered (1 GPU runs only)
* ``c5a``        1024 sequences x 8192 keys split over the N ranks (strong scaling, no collective)
* ``c5b``        one 131072-token sequence, KV heads split over the N ranks + one NCCL all-gather
* ``sustained``  c2 steps back to back for at least two seconds, with the clocks seen
* ``module_path``  the same c2 decode driven through ``AttentionB200`` + ``PagedKVCache``

* ``value``     decode tokens/s, whole job, inputs resident in HBM (CUDA events, max over ranks).
* ``e2e``       the same step driven from pinned HOST buffers through ``GraphedDecodeStep``: q / new K,V /
                slot mapping / lengths copied in, result copied out, every step.
* ``roofline``  algorithmic bytes of the attention call / its mean duration, against the measured
                HBM copy bandwidth of this pool's B200s.
* ``cpu_baseline``  the CPU checker (the reference's torch path restated) timed on the host cores.
"""

from __future__ import annotations

import argparse
import gc
import json
import math
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
# c2: 8-sequence case, 539.11 MB read + 4.06 MB written (mean of two launches) for 537.14 MB algorithmic;
# c3: 32-sequence case, 350.44 MB + 4.98 MB for 349.93 MB.  Traffic grows with the tokens read, so the
# ratio carries over to the full-size launch.
NCU_TRAFFIC_RATIO = {"c2": (539.11 + 4.06) / 537.14, "c3": (350.44 + 4.98) / 349.93, "c5a": (350.44 + 4.98) / 349.93}


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


def roofline_record(nbytes, ms, kernel=None, traffic_ratio=None):
    peak, kind = measured_peak()
    achieved = nbytes / (ms * 1e-3) / 1e9
    rec = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
           "peak_kind": f"of {kind}", "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
           "algorithmic_bytes": int(nbytes), "ms": ms,
           "traffic": None if traffic_ratio is None else int(nbytes * traffic_ratio)}
    if kernel:
        rec["kernel"] = kernel
    return rec


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

    def mark(self):
        """Index of the next sample (to summarise a sub-interval later)."""
        return len(self.rows)

    def summary(self, start=0, stop=None):
        rows = self.rows[start:stop]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]

        def num(x):
            try:
                return float(x)
            except ValueError:
                return None

        power = [num(r[6]) for r in rows if len(r) > 6 and num(r[6]) is not None]
        mem = [num(r[7]) for r in rows if len(r) > 7 and num(r[7]) is not None]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_min_mhz": min(int(r[0]) for r in rows),
                "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows),
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
    """Lengths and head layout of a workload without building its pools."""
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


# ---- timing helpers -----------------------------------------------------------------------------------

def time_region(fn, steps, flush=None):
    """CUDA-event time of ``steps`` calls on the current stream, in ms (one event pair per call so
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


class Ranks:
    """The process group (if any) and the max-over-ranks reduction every multi-GPU figure goes through."""

    def __init__(self, dev):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.dev = dev
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            # whatever NCCL logs (its version banner, for one) goes to stderr: stdout carries the one JSON line
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
            dist.init_process_group("nccl", device_id=dev)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max(self, *values):
        if self.dist is None:
            return values if len(values) > 1 else values[0]
        t = torch.tensor(list(values), device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        out = [float(v) for v in t.tolist()]
        return out if len(out) > 1 else out[0]

    def close(self):
        if self.dist is not None:
            self.dist.barrier()
            self.dist.destroy_process_group()


def quantise_pools(wl, dev):
    """--kv-fp8: replace the 16-bit pools by e4m3 pools (N(0,1) data, scale 1/64 keeps +-7 sigma in range)."""
    for attr in ("k_pool", "v_pool"):
        pool = getattr(wl, attr)
        q8 = torch.empty(pool.shape, dtype=torch.float8_e4m3fn, device=dev)
        step_rows = 1 << 16
        for lo in range(0, pool.shape[2], step_rows):      # chunked: no full-size fp32 temporary
            q8[:, :, lo:lo + step_rows] = (pool[:, :, lo:lo + step_rows].float() * 64.0).clamp(-448, 448).to(torch.float8_e4m3fn)
        setattr(wl, attr, q8)
    torch.cuda.empty_cache()
    return {"k_scale": 1.0 / 64, "v_scale": 1.0 / 64}


_flush_bufs = {}


def flusher(dev, nbytes_read=0, always=False):
    """An L2 flush for workloads whose K/V would otherwise stay cached: 512 MB are written (the L2 holds
    126 MB) and then read back.  The read pass matters for short kernels: a write-only flush leaves the
    L2 full of DIRTY lines, and the next kernel pays for writing ~126 MB back to HBM while it runs (about
    20 us of HBM time -- measured: 10 % on a 100 us kernel); after the read pass the L2 holds clean lines of
    the flush buffer and nothing of the workload.  ``always``: also for legs whose GPU time per call is
    shorter than the host's launch cost -- the ~170 us of flush keep the host ahead of the GPU, so the
    event pair around the call measures the device and not the launch path."""
    if nbytes_read > 4 * 126e6 and not always:
        return None, None
    buf = _flush_bufs.get(dev)
    if buf is None:
        buf = _flush_bufs[dev] = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def flush():
        buf.fill_(1)
        buf.view(torch.int64).max()

    return buf, flush


def graph_of(fn, dev):
    """``fn`` recorded as a CUDA graph (after one eager run on a side stream, which does the kernels'
    one-time set-up outside the capture); returns the replay callable."""
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        fn()
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        fn()
    return graph.replay


# ---- decode workloads (c2, c3, c5a) ----------------------------------------------------------------------

def measure_decode(name, wl, ranks, steps, warmup, kv_scales, seqs_total):
    """Device-resident timing of the decode step (paged_decode_step: append + attention in one call) on one
    decode workload, plus the attention call and the stand-alone append kernel on their own.  Returns a dict
    with the whole step (max over ranks) and the per-kernel legs of this rank."""
    dev = ranks.dev
    lib = iva_b200.load_library()
    B = wl.batch
    lens = (wl.ctx_len + wl.new_tokens_per_seq).contiguous()
    out = torch.empty(B, wl.n_q_heads, wl.head_dim, device=dev, dtype=wl.dtype)
    lse = torch.empty(B, wl.n_q_heads, device=dev, dtype=torch.float32)
    nbytes = attention_bytes(wl, lens)
    flush_buf, flush = flusher(dev, nbytes)

    def append():
        iva_b200.paged_append(wl.k_pool, wl.v_pool, wl.slot_mapping, wl.k_new, wl.v_new, wl.page_size, **kv_scales)

    def attend():
        iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, wl.page_size, wl.scale,
                                        out=out, lse=lse, **kv_scales)

    def step():
        # the decode step as one call: the new token of every sequence is written by the attention launch
        iva_b200.paged_decode_step(wl.q, wl.k_new, wl.v_new, wl.k_pool, wl.v_pool, wl.block_table, lens, wl.page_size,
                                   wl.scale, out=out, lse=lse, **kv_scales)

    for _ in range(max(warmup, 3)):
        step()
    ranks.barrier()
    launches0 = lib.ivab_launch_count()
    per_step = time_region(step, steps, flush)
    ranks.barrier()
    launches = lib.ivab_launch_count() - launches0
    attn_ms = time_region(attend, steps, flush)
    app_ms = time_region(append, steps, flusher(dev, always=True)[1])   # microseconds of GPU time: keep the host ahead
    total_ms = ranks.max(sum(per_step))
    ms_per_step = total_ms / steps
    rec = {"ms_per_step": ms_per_step, "value": seqs_total * wl.new_tokens_per_seq / (ms_per_step * 1e-3),
           "unit": "decode tok/s", "attention_ms": statistics.mean(attn_ms), "attention_ms_min": min(attn_ms),
           "append_ms": statistics.mean(app_ms), "append_GBs": append_bytes(wl) / (statistics.mean(app_ms) * 1e-3) / 1e9,
           "gpu_launches": int(launches), "l2": "flushed between timed steps" if flush else "K/V per step exceed L2",
           "roofline": roofline_record(nbytes, statistics.mean(attn_ms),
                                       "plan_kernel + decode_kernel + merge_kernel (one attention call)",
                                       NCU_TRAFFIC_RATIO.get(name))}
    return rec, step, out, lens


def measure_sustained(step, batch, ranks, clocks, ms_per_step, seconds=2.5):
    """Steps back to back for a few seconds: the figure a long-running server sees, with the clocks and
    power-cap state sampled over exactly this interval."""
    n = max(50, int(math.ceil(seconds * 1e3 / ms_per_step)))
    ranks.barrier()
    m0 = clocks.mark()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        step()
    b.record()
    torch.cuda.synchronize()
    time.sleep(0.06)
    m1 = clocks.mark()
    ms = ranks.max(a.elapsed_time(b))
    ranks.barrier()
    c = clocks.summary(m0, m1)
    rec = {"steps": n, "seconds": ms * 1e-3, "ms_per_step": ms / n, "value": batch * ranks.world / (ms / n * 1e-3),
           "unit": "decode tok/s", "clocks": c}
    if c.get("sm_mhz"):
        rec["ms_per_step_x_sm_ghz"] = ms / n * c["sm_mhz"] * 1e-3      # clock-normalised: compare across runs
    return rec


def measure_e2e(wl, lens, ranks, steps, warmup, kv_scales, seqs_total, out_check=None):
    """The public end-to-end call: inputs in pinned host memory, one CUDA-graph replay per step (H2D of
    q / new K,V / slot mapping / lengths, append, attention; the kernels store the output straight into
    the pinned host buffer, d2h_bytes_per_step counts those bytes).

    ``value``: one batch, strictly serial -- the host waits for step k's output before it enqueues step
    k+1, as a decode loop must (the next query depends on it).  ``two_batches_in_flight``: two independent
    copies of the batch (own pools, own stream) alternate, each still waiting for its own previous output;
    one batch's upload and host turn-around hide under the other's attention."""
    def make(k_pool, v_pool, **kw):
        gs = iva_b200.GraphedDecodeStep(k_pool, v_pool, wl.block_table, wl.n_q_heads, wl.page_size, wl.scale,
                                        token_dtype=wl.dtype, **kv_scales, **kw)
        for b in range(gs.n_buffers):
            io = gs.inputs(b)
            io.q_host.copy_(wl.q)
            io.k_new_host.copy_(wl.k_new)
            io.v_new_host.copy_(wl.v_new)
            io.slot_mapping_host.copy_(wl.slot_mapping)
            io.ctx_len_host.copy_(lens)
        return gs

    gs = make(wl.k_pool, wl.v_pool)
    torch.cuda.synchronize()

    def e2e_step():
        gs.run(0)
        return gs.result(0)                                # the host consumes the result every step

    for _ in range(max(warmup, 3)):
        e2e_step()
    ranks.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        res = e2e_step()
    torch.cuda.synchronize()
    wall_ms = ranks.max((time.perf_counter() - t0) * 1e3)
    if out_check is not None:
        assert torch.equal(res.to(out_check.device), out_check), "end-to-end result differs from the device-resident one"
    rec = {"value": seqs_total / (wall_ms / steps * 1e-3), "unit": "decode tok/s",
           "h2d_bytes_per_step": gs.h2d_bytes, "d2h_bytes_per_step": gs.d2h_bytes,
           "ms_per_step": wall_ms / steps,
           "api": "GraphedDecodeStep.run() + result(): host clock around K steps; the host waits for each step's "
                  "output (an event behind its last kernel) before it enqueues the next"}

    # the same serial loop without the upload: the kernels read q, the new tokens and the lengths from the pinned
    # staging block in place (the bytes still cross the bus every step, under the attention kernel instead of
    # in front of it; q rows are read once per chunk of their sequence, so somewhat more of them)
    gz = make(wl.k_pool, wl.v_pool, zero_copy_inputs=True)
    for _ in range(max(warmup, 3)):
        gz.run(0)
        gz.result(0)
    ranks.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        gz.run(0)
        resz = gz.result(0)
    torch.cuda.synchronize()
    wallz = ranks.max((time.perf_counter() - t0) * 1e3)
    rec["inputs_read_in_place"] = {"value": seqs_total / (wallz / steps * 1e-3), "unit": "decode tok/s",
                                   "ms_per_step": wallz / steps, "same_bits": bool(torch.equal(resz, res)),
                                   "note": "GraphedDecodeStep(zero_copy_inputs=True): no host->device copy node; the "
                                           "kernels load the step's inputs from pinned host memory while they run"}
    del gz

    # two independent batches in flight
    free, _ = torch.cuda.mem_get_info()
    need = 2 * wl.k_pool.numel() * wl.k_pool.element_size()
    if free > need + (8 << 30):
        gs2 = make(wl.k_pool.clone(), wl.v_pool.clone())
        pair = (gs, gs2)
        for g in pair:
            g.run(0)
            g.result(0)
        ranks.barrier()
        t0 = time.perf_counter()
        for g in pair:
            g.run(0)
        for _ in range(steps):
            for g in pair:
                g.result(0)
                g.run(0)
        for g in pair:
            g.result(0)
        wall2 = ranks.max((time.perf_counter() - t0) * 1e3)
        n_steps = 2 * (steps + 1)
        rec["two_batches_in_flight"] = {
            "value": (seqs_total * n_steps) / (wall2 * 1e-3), "unit": "decode tok/s", "ms_per_batch_step": wall2 / n_steps,
            "note": "two independent batches of this configuration (own pools, own stream) alternate; each batch "
                    "still reads its own step-k output before its step k+1 is enqueued"}
        assert torch.equal(gs2.result(0), gs.result(0))
        del gs2
    return rec


def measure_module_path(dev, ranks, steps, warmup):
    """c2 decode through the drop-in module contract: ``AttentionB200.forward(x, kv_cache=PagedKVCache)``
    with real bias-free projections (d_model 4096), 64 sequences at context 4096 growing by one token per
    step.  ``value`` is pipelined (the layer's output stays on the device, as inside a model; one
    synchronisation at the end); ``synced`` forces the host to wait for every step."""
    from types import SimpleNamespace
    B, H, D, ctx = 64, 32, 128, 4096
    cfg = SimpleNamespace(d_model=H * D, n_heads=H, dropout=0.0, causal=False, attn_impl="b200")
    mod = iva_b200.AttentionB200(cfg).to(device=dev, dtype=torch.bfloat16).eval()
    n_total = 2 * (steps + max(warmup, 3)) + 8
    cache = iva_b200.PagedKVCache(batch_size=B, n_heads=H, head_dim=D, seq_len=ctx, device=dev, dtype=torch.bfloat16,
                                  max_seq_len=ctx + n_total, shuffle_seed=1)
    cache.k_pool.normal_()
    cache.v_pool.normal_()
    x = torch.randn(B, 1, H * D, device=dev, dtype=torch.bfloat16)

    def proj_only():
        mod.o_proj(mod.q_proj(x) + mod.k_proj(x) + mod.v_proj(x))

    def step():
        y, _ = mod(x, kv_cache=cache)
        return y

    for _ in range(max(warmup, 3)):
        step()
    ranks.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        y = step()
    torch.cuda.synchronize()
    pipelined = (time.perf_counter() - t0) * 1e3 / steps
    t0 = time.perf_counter()
    for _ in range(steps):
        y = step()
        torch.cuda.current_stream().synchronize()
    synced = (time.perf_counter() - t0) * 1e3 / steps
    proj = statistics.mean(time_region(proj_only, steps))
    pipelined, synced = ranks.max(pipelined, synced)
    assert torch.isfinite(y.float()).all()
    return {"value": B * ranks.world / (pipelined * 1e-3), "unit": "decode tok/s", "ms_per_step": pipelined,
            "synced": {"value": B * ranks.world / (synced * 1e-3), "ms_per_step": synced},
            "projections_ms": proj, "context_at_end": cache.seq_len,
            "api": "AttentionB200.forward(x [64,1,4096] bf16, kv_cache=PagedKVCache): q/k/v projections, paged append, "
                   "paged decode attention, o projection; host clock around K steps"}


# ---- c4: append / gather stress ----------------------------------------------------------------------

def measure_c4(wl, ranks, steps, warmup):
    dev = ranks.dev
    B = wl.batch
    lens = (wl.ctx_len + wl.new_tokens_per_seq).contiguous()
    offs = torch.zeros(B + 1, dtype=torch.int64, device=dev)
    offs[1:] = torch.cumsum(lens.long(), 0)
    total_tokens = int(offs[-1])

    def append():
        iva_b200.paged_append(wl.k_pool, wl.v_pool, wl.slot_mapping, wl.k_new, wl.v_new, wl.page_size)

    def gather():
        k = iva_b200.paged_gather(wl.k_pool, wl.block_table, lens, wl.page_size, layout="token_major",
                                  out_offsets=offs, total_tokens=total_tokens)
        v = iva_b200.paged_gather(wl.v_pool, wl.block_table, lens, wl.page_size, layout="token_major",
                                  out_offsets=offs, total_tokens=total_tokens)
        return k, v

    for _ in range(max(warmup, 3)):
        append()
    gather()
    ranks.barrier()
    app_ms = time_region(append, steps)
    gat_ms = time_region(gather, max(3, steps // 4))
    app, gat = statistics.mean(app_ms), statistics.mean(gat_ms)
    return {"tokens_appended": int(wl.k_new.shape[0]), "tokens_gathered": total_tokens,
            "append": roofline_record(append_bytes(wl), app, "row_copy_kernel<scatter> (K and V in one launch)"),
            "gather": roofline_record(gather_bytes(wl, lens), gat, "paged_gather_kernel (K, then V)"),
            "append_ms_min": min(app_ms), "gather_ms_min": min(gat_ms),
            "note": "a copy cannot exceed the measured copy bandwidth of the part (the 'peak' above), which is "
                    "0.81 of the nominal 8 TB/s; frac_of_nominal_8TBs is therefore capped near 0.81-0.83"}


# ---- c5b: head-parallel decode of one long sequence ---------------------------------------------------------

def measure_c5b(wl, ranks, steps, warmup, use_graph=True, exchange="nccl"):
    from iva_b200.sharding import HeadParallelDecoder
    dev = ranks.dev
    world = ranks.world
    lens = (wl.ctx_len + 1).contiguous()
    nbytes = attention_bytes(wl, lens) // world
    if world > 1:
        hp = HeadParallelDecoder(wl.n_q_heads, wl.n_kv_heads, exchange=exchange)
        k_loc, v_loc = hp.local_pools(wl.k_pool, wl.v_pool)
        k_loc, v_loc = k_loc.contiguous(), v_loc.contiguous()          # each rank keeps only its slab
        k_new, v_new = wl.k_new[:, hp.kv_slice].contiguous(), wl.v_new[:, hp.kv_slice].contiguous()
    else:
        hp = None
        k_loc, v_loc, k_new, v_new = wl.k_pool, wl.v_pool, wl.k_new, wl.v_new
    flush_buf, flush_local = flusher(dev, nbytes, always=True)   # a step is ~0.1 ms or less: see flusher()
    if world > 1:
        # The flush takes a different time on every GPU, and a step that ends in a collective would charge
        # that skew to whichever rank finished its flush first.  A one-word all-reduce behind the flush
        # (outside the timed region; issued twice) lets the ranks start each timed step together, as they do in a decode
        # loop, where the previous step's collective has aligned them.
        sync_word = torch.zeros(1, device=dev)

        def flush():
            flush_local()
            ranks.dist.all_reduce(sync_word)   # absorbs the skew of the flush ...
            ranks.dist.all_reduce(sync_word)   # ... and this one starts, and so ends, nearly together on all ranks
    else:
        flush = flush_local

    def append():
        iva_b200.paged_append(k_loc, v_loc, wl.slot_mapping, k_new, v_new, wl.page_size)

    if hp is not None:
        hp_attn = hp.capture_local(wl.q, k_loc, v_loc, wl.block_table, lens, wl.page_size, wl.scale) if use_graph else None
        # the whole step (append + attention) as one graph replay, followed by the one eager all-gather
        hp_step = (hp.capture_local(wl.q, k_loc, v_loc, wl.block_table, lens, wl.page_size, wl.scale,
                                    new_tokens=(k_new, v_new)) if use_graph else None)

        def attend():
            if hp_attn is not None:
                return hp_attn()
            return hp.decode(wl.q, k_loc, v_loc, wl.block_table, lens, wl.page_size, wl.scale)
    else:
        out = torch.empty(1, wl.n_q_heads, wl.head_dim, device=dev, dtype=wl.dtype)
        lse = torch.empty(1, wl.n_q_heads, device=dev, dtype=torch.float32)
        ws = torch.empty(iva_b200.decode_workspace_bytes(1, wl.n_q_heads, wl.n_kv_heads, wl.head_dim), dtype=torch.uint8,
                         device=dev)

        def attend():
            return iva_b200.paged_decode_attention(wl.q, k_loc, v_loc, wl.block_table, lens, wl.page_size, wl.scale,
                                                   out=out, lse=lse, workspace=ws)

        def both():
            iva_b200.paged_decode_step(wl.q, k_new, v_new, k_loc, v_loc, wl.block_table, lens, wl.page_size, wl.scale,
                                       out=out, lse=lse, workspace=ws)

        # one GPU: the same step as one graph replay (a step of ~0.1 ms is launch-bound when issued from Python)
        hp_step = graph_of(both, dev) if use_graph else None

    def local_only():
        iva_b200.paged_decode_attention(wl.q[:, hp.q_slice] if hp is not None else wl.q, k_loc, v_loc, wl.block_table,
                                        lens, wl.page_size, wl.scale, return_lse=True)

    def step():
        if hp_step is not None:
            return hp_step()
        append()
        return attend()

    for _ in range(max(warmup, 3)):
        step()
    ranks.barrier()
    per_step = time_region(step, steps, flush)
    ranks.barrier()
    attn_ms = time_region(attend, steps, flush)          # local kernels + the all-gather
    kern_ms = time_region(local_only, steps, flush)      # this rank's attention kernels only
    ms_per_step = ranks.max(sum(per_step)) / steps
    attn, kern = ranks.max(statistics.mean(attn_ms), statistics.mean(kern_ms))
    eager_ms = None
    if hp is not None and exchange == "p2p":
        # the same step launched eagerly (one library call; this measurement's flush keeps the host ahead of the GPU)
        eager_step = hp.capture_local(wl.q, k_loc, v_loc, wl.block_table, lens, wl.page_size, wl.scale,
                                      new_tokens=(k_new, v_new), graph=False)
        for _ in range(3):
            eager_step()
        ranks.barrier()
        eager_ms = ranks.max(sum(time_region(eager_step, steps, flush))) / steps
    # what the step returned (all ranks' rows on this rank): both exchange methods must give the same bits
    res = step()
    if not isinstance(res, tuple):      # one GPU: the graph replay wrote into out / lse
        res = (out, lse)
    torch.cuda.synchronize()
    import hashlib
    digest = hashlib.sha1(b"".join(t.detach().float().cpu().contiguous().numpy().tobytes() for t in res)).hexdigest()[:16]
    return {"ms_per_step": ms_per_step, "result_digest": digest, "ms_per_step_eager_launch": eager_ms, "attention_incl_allgather_ms": attn, "attention_kernels_ms": kern,
            "value": 1.0 / (ms_per_step * 1e-3), "unit": "decode tok/s (one sequence)",
            "roofline_local_kernels": roofline_record(nbytes, kern, "this rank's plan + decode + merge kernels"),
            "kv_heads_per_rank": wl.n_kv_heads // world, "collective": None if world == 1 else (
                "one NCCL all_gather_into_tensor of [1, H_q/N, D+1] fp32 per step (eager; local kernels in a CUDA graph)"
                if exchange == "nccl" else
                "ivab_paged_decode_step_allgather: the merge kernel's last CTA sends this rank's rows to the peers over NVLink "
                "({payload, step tag} words into peer-mapped memory, no fence) and collects theirs; one graph replay per step, "
                "no exchange launch, no NCCL call"),
            "l2": "flushed between timed steps" + ("; ranks aligned by a one-word all-reduce behind each flush, "
                                                    "outside the timed region" if world > 1 else "")}


# ---- the GPU arm --------------------------------------------------------------------------------------

def free_gpu(*objs):
    del objs
    gc.collect()
    torch.cuda.empty_cache()


def run_gpu(args):
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    if world_env != args.gpus and world_env == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ranks = Ranks(dev)
    world, rank = ranks.world, ranks.rank
    iva_b200.load_library()
    name = "c2" if args.workload == "all" else args.workload
    everything = args.workload == "all"
    copy_gbs = live_copy_bandwidth(dev)
    clocks = ClockSampler(local)
    clocks.__enter__()
    result = None

    if name in ("c2", "c3", "c5a"):
        wl = build_workload(name, dev, rank, world, args)
        kv_scales = quantise_pools(wl, dev) if args.kv_fp8 else {}
        seqs_total = wl.batch * world
        rec, step, out, lens = measure_decode(name, wl, ranks, args.steps, args.warmup, kv_scales, seqs_total)
        m_end = clocks.mark()
        e2e = measure_e2e(wl, lens, ranks, args.steps, args.warmup, kv_scales, seqs_total, out_check=out)
        sustained = measure_sustained(step, wl.batch, ranks, clocks, rec["ms_per_step"]) if everything or args.sustained else None
        roof = rec.pop("roofline")
        roof.update({"live_copy_GBs_this_gpu": copy_gbs, "frac_of_live_copy": roof["achieved"] / copy_gbs})
        result = {
            "metric": METRIC, "value": rec["value"], "unit": "decode tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if name == "c5a" else "weak", "vs_baseline": None,
            "dtype": {"torch.bfloat16": "bf16", "torch.float16": "f16", "torch.float32": "f32"}[str(wl.dtype)],
            "data": "synthetic (seeded N(0,1) K/V/q, shuffled page pool)",
            "config": describe(name, args, rank, world, args.kv_fp8),
            "roofline": roof,
            "kernels": {k: rec[k] for k in ("append_ms", "append_GBs", "attention_ms", "attention_ms_min")},
            "e2e": e2e, "gpu_launches": rec["gpu_launches"],
        }
        if sustained is not None:
            result["sustained"] = sustained
        del wl, step, out, lens
        free_gpu()
        if everything:
            result["module_path"] = measure_module_path(dev, ranks, args.steps, args.warmup)
            free_gpu()
    elif name == "c4":
        wl = build_workload("c4", dev, rank, world, args)
        c4 = measure_c4(wl, ranks, args.steps, args.warmup)
        result = {"metric": METRIC, "value": c4["gather"]["achieved"], "unit": "GB/s (paged gather)", "n_gpus": world,
                  "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": c4["gather"]["ms"] + c4["append"]["ms"],
                  "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
                  "data": "synthetic (seeded N(0,1) K/V, shuffled page pool)", "config": describe("c4", args, rank, world),
                  "roofline": c4["gather"], "c4": c4, "gpu_launches": 3 * args.steps}
        del wl
        free_gpu()
    else:   # c5b alone
        wl = build_workload("c5b", dev, rank, world, args)
        c5b = measure_c5b(wl, ranks, args.steps, args.warmup, use_graph=not args.no_graph)
        result = {"metric": METRIC, "value": c5b["value"], "unit": c5b["unit"], "n_gpus": world, "steps": args.steps,
                  "warmup": max(args.warmup, 3), "ms_per_step": c5b["ms_per_step"], "higher_is_better": True,
                  "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                  "data": "synthetic (seeded N(0,1) K/V/q, shuffled page pool)", "config": describe("c5b", args, rank, world),
                  "roofline": c5b["roofline_local_kernels"], "c5b": c5b, "gpu_launches": 4 * args.steps}
        del wl
        free_gpu()

    if everything:
        sub_steps = max(10, min(args.steps, 30))
        if world == 1:
            wl = build_workload("c3", dev, rank, world, args)
            rec, _, _, _ = measure_decode("c3", wl, ranks, sub_steps, args.warmup, {}, wl.batch)
            rec["config"] = describe("c3", args, rank, world)
            result["c3"] = rec
            del wl
            free_gpu()
            wl = build_workload("c4", dev, rank, world, args)
            result["c4"] = measure_c4(wl, ranks, sub_steps, args.warmup)
            del wl
            free_gpu()
        wl = build_workload("c5a", dev, rank, world, args)
        rec, _, _, _ = measure_decode("c5a", wl, ranks, sub_steps, args.warmup, {}, wl.batch * world)
        rec["config"] = describe("c5a", args, rank, world)
        rec["scaling"] = "strong: 1024 sequences x 8192 keys split evenly over the ranks, slowest rank's time"
        result["c5a"] = rec
        del wl
        free_gpu()
        wl = build_workload("c5b", dev, rank, world, args)
        result["c5b"] = measure_c5b(wl, ranks, sub_steps, args.warmup, use_graph=not args.no_graph)
        if world > 1:
            # the same step with the outputs reassembled by the library's own kernel over peer memory
            try:
                p2p = measure_c5b(wl, ranks, sub_steps, args.warmup, use_graph=not args.no_graph, exchange="p2p")
                result["c5b"]["peer_memory_exchange"] = {"same_bits_as_nccl": p2p["result_digest"] == result["c5b"]["result_digest"]}
                result["c5b"]["peer_memory_exchange"].update({k: p2p[k] for k in ("ms_per_step", "ms_per_step_eager_launch", "attention_incl_allgather_ms",
                                                                                 "value", "collective")})
            except Exception as e:                      # (symmetric memory not available on this system)
                result["c5b"]["peer_memory_exchange"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        del wl
        free_gpu()

    clocks.__exit__(None, None, None)
    result["clocks"] = clocks.summary()
    if rank != 0:
        ranks.close()
        return
    if args.cpu_baseline and world == 1:
        result["cpu_baseline"] = cpu_baseline(name, args, budget_s=12.0)
        result["c1_reference_case"] = c1_case(dev)
    print(json.dumps(result))
    ranks.close()


# ---- the CPU arm (checker timed as a baseline) ------------------------------------------------------------

def cpu_sample(name, args, full):
    """The CPU arm's workload: the whole configuration when the host can hold it, else a bounded sample
    of it (same heads, dtype, page size and contexts, fewer sequences)."""
    if name == "c3":
        return workloads.config_c3(device="cpu", batch=8), "8 of 128 sequences (same length distribution)"
    if name == "c5a":
        return workloads.config_c5a(device="cpu", n_seq=2, context=args.context or 8192), "2 of 1024 sequences"
    if name == "c5b":
        return workloads.config_c5b(device="cpu", context=16384), "one sequence cut to 16384 tokens"
    ctx = args.context or 4096
    batch = args.batch or 64
    if full:
        return workloads.config_c2(device="cpu", batch=batch, context=ctx), f"all {batch} sequences, context {ctx}"
    return workloads.config_c2(device="cpu", batch=4, context=ctx), f"4 of {batch} sequences, context {ctx}, own pool"


def host_can_hold_full_c2(args):
    """The full c2 step on the host needs the two pools (4.3 GB) and their clones inside the restated
    scatter (another 4.3 GB) plus fp32 temporaries: ask for 24 GB of free memory."""
    try:
        import psutil
        return psutil.virtual_memory().available > 24 * (1 << 30) * max(1, (args.batch or 64) * (args.context or 4096)) / (64 * 4096)
    except Exception:
        return False


def cpu_baseline(name, args, budget_s, kind_label="port", full=False, exact_steps=None):
    from oracle import paged_ref as ref

    torch.set_num_threads(os.cpu_count() or 1)
    wl, sample = cpu_sample(name if name != "c4" else "c2", args, full)
    t0 = time.perf_counter()
    ref.decode_step_ref(wl)                                    # warm-up
    first = time.perf_counter() - t0
    times = []
    if exact_steps is not None:
        warm, k = exact_steps
        # keep the whole run within a few minutes: cut the step count if a step is slower than expected
        k = max(3, min(k, int(240.0 / max(first, 1e-3))))
        for _ in range(max(0, warm - 1)):
            ref.decode_step_ref(wl)
        for _ in range(k):
            t0 = time.perf_counter()
            ref.decode_step_ref(wl)
            times.append(time.perf_counter() - t0)
    else:
        t_end = time.perf_counter() + budget_s
        while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 200):
            t0 = time.perf_counter()
            ref.decode_step_ref(wl)
            times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": wl.batch / med, "unit": "decode tok/s", "cores": torch.get_num_threads(), "kind": kind_label,
            "sample": f"{sample}; median of {len(times)} steps of the torch-CPU restatement of the reference path "
                      f"(clone+index_copy append, index_select gather, matmul/softmax/matmul)",
            "sample_batch": wl.batch, "timed_steps": len(times),
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
    _, flush = flusher(dev, always=True)

    def step():
        iva_b200.paged_append(d.k_pool, d.v_pool, d.slot_mapping, d.k_new, d.v_new, wl.page_size)
        iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, lens, wl.page_size, wl.scale, out=out)

    for _ in range(5):
        step()
    gpu = time_region(step, 50, flush)
    # the same two calls replayed as one CUDA graph (what a serving loop does with a launch-bound step)
    ws = torch.empty(iva_b200.decode_workspace_bytes(wl.batch, wl.n_q_heads, wl.n_kv_heads, wl.head_dim), dtype=torch.uint8,
                     device=dev)

    def graphed():
        iva_b200.paged_decode_step(d.q, d.k_new, d.v_new, d.k_pool, d.v_pool, d.block_table, lens, wl.page_size, wl.scale,
                                   out=out, workspace=ws)

    replay = graph_of(graphed, dev)
    for _ in range(5):
        replay()
    gpu_graph = time_region(replay, 200, flush)     # (event pairs resolve ~2 us here: the mean of many is the figure)
    nbytes = attention_bytes(wl, wl.ctx_len + 1) + append_bytes(wl)
    return {"config": "batch 4, 16 heads, head_dim 64, fp32, contexts " + str(wl.ctx_len.tolist()),
            "cpu_ms_per_step": statistics.median(cpu) * 1e3, "cpu_cores": torch.get_num_threads(),
            "gpu_ms_per_step": statistics.median(gpu), "gpu_ms_per_step_graph_replay": statistics.mean(gpu_graph),
            "gpu_ms_per_step_graph_replay_median": statistics.median(gpu_graph),
            "algorithmic_bytes": nbytes,
            "note": "latency-bound on the GPU: 1 MB of K/V; the graph replay is the device time (two kernels), the "
                    "eager figure includes what the Python launch path adds when the GPU is faster than the host"}


def run_reference(args):
    """``--impl reference``: the reference's own path on the host cores.  The reference is pure
    Python whose package cannot be imported (syntax errors in three of its modules) and is not present
    where this benchmark runs, so the timed code is the checker's restatement of it on PyTorch CPU
    operators -- on the whole configuration when the host's memory allows, else on a sample of it that
    the line names."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = "c2" if args.workload == "all" else args.workload
    full = name in ("c2", "c4") and host_can_hold_full_c2(args)
    base = cpu_baseline(name, args, budget_s=0.0, full=full, exact_steps=(args.warmup, args.steps))
    wl_dtype = "f16" if name == "c4" else "bf16"
    cfg = describe(name, args, 0, 1)
    cfg["timed_batch"] = base["sample_batch"]
    cfg["timed"] = base["sample"]
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "decode tok/s",
        "n_gpus": args.gpus, "steps": base["timed_steps"], "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl_dtype,
        "data": "synthetic (seeded N(0,1) K/V/q, shuffled page pool)", "config": cfg,
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
    ap.add_argument("--workload", default="all", choices=["all", "c2", "c3", "c4", "c5a", "c5b"],
                    help="all = the c2 headline plus one sub-record per other configuration")
    ap.add_argument("--batch", type=int, default=0, help="override the number of sequences (small ncu captures)")
    ap.add_argument("--context", type=int, default=0, help="override the context length")
    ap.add_argument("--no-cpu-baseline", dest="cpu_baseline", action="store_false")
    ap.add_argument("--kv-fp8", action="store_true", help="store K/V as e4m3 with per-tensor scales (c2/c3/c5a)")
    ap.add_argument("--sustained", action="store_true", help="add the seconds-long leg to a single-workload run")
    ap.add_argument("--no-graph", action="store_true", help="head-parallel mode: launch eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
