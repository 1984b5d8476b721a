"""Benchmark of the hot path: batch-sharded inference forward of the 784-1024-1024-10 MLP.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One process per GPU (the launcher is torch.distributed.run for N > 1).  ONE batch of `--rows`
rows (8192 x 784) is split along its leading axis into N contiguous shards, as
`Parallel.shard_along` does (lib/parallel.ml:51-66); every rank runs the forward routine over its
shard (strong scaling, no data-path collective — inference forward shards by batch).  A step =
one run of the routine over one batch.  The weak-scaling figure (every GPU keeps all `--rows`
rows) is reported beside it as `weak`.

Reported on ONE JSON line by rank 0:
  value      forward samples/s of the whole job, inputs resident in device memory
  e2e        the same through the host-facing calls: page-locked host batch -> from_host ->
             run -> to_host of the loss, copies inside the timed region
  roofline   the dominant kernel (the widest hidden-layer contraction): algorithmic FLOPs /
             its CUDA-event duration, against the measured bf16 peak
             `roofline.contraction` holds config 3 (`b|m,k ; b|k,n => b|m,n` + bias + GELU, batch 8)
             at 1024 / 4096 / 8192: kernel ms, TFLOP/s, fraction of the measured bf16 peak
  cpu_baseline  the restated cc backend (oracle) on one host core over the same shard; its loss
             is what the device's loss is checked against
Timing: per-step CUDA events on the library's stream, L2 flushed between steps by clearing a
256 MiB buffer outside the timed events; the job time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# stdout carries the one JSON line and nothing else: when the environment asks NCCL for
# diagnostics (NCCL_DEBUG), they go to stderr instead of NCCL's default, stdout
if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
    # this level prints one line, "NCCL version ...", on stdout at the first communicator
    del os.environ["NCCL_DEBUG"]
    _NCCL_VERSION_WANTED = True
else:
    _NCCL_VERSION_WANTED = False
    if os.environ.get("NCCL_DEBUG") and not os.environ.get("NCCL_DEBUG_FILE"):
        os.environ["NCCL_DEBUG_FILE"] = "/dev/stderr"

METRIC = "forward samples/sec"
WORKLOAD = ("config 5 forward: MLP 784-1024-1024-10, bf16 weights and activations, fp32 accumulation, softmax "
            "cross-entropy; ONE [%d, 784] batch split by rows over the GPUs, no collective")
DIMS = (784, 1024, 1024, 10)


_T0 = time.time()


def progress(msg):
    """One line per phase on stderr (stdout carries the JSON line only)."""
    print("[bench %6.1fs rank %s] %s" % (time.time() - _T0, os.environ.get("RANK", "0"), msg), file=sys.stderr, flush=True)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"bf16": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"], "hbm": d["hbm_gbs"],
                "source": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML read-outs every
    millisecond from a thread (reading only; nothing is set), nvidia-smi as the fallback."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index = index
        self.sm, self.mask, self.max_mhz = [], 0, None
        self.stop_flag = threading.Event()
        self.thread = None
        self.nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nvml = None
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nvml
        reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                self.mask |= int(reasons(self.handle))
            except Exception:
                break
            time.sleep(0.001)

    def stop(self):
        self.stop_flag.set()
        if self.thread:
            self.thread.join(timeout=2)
        if self.sm:
            return {"sm_mhz": float(np.median(self.sm)), "sm_max_mhz": self.max_mhz,
                    "reasons": [n for bit, n in self.REASONS.items() if self.mask & bit], "samples": len(self.sm),
                    "source": "NVML, 1 ms period, from warm-up to the end of the end-to-end steps"}
        # fallback: one nvidia-smi reading
        try:
            q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
            out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                  "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=20).stdout
            rows = [[c.strip() for c in line.split(",")] for line in out.splitlines() if line.strip()]
        except (OSError, subprocess.SubprocessError):
            rows = []
        sm = [float(r[0]) for r in rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "source": "nvidia-smi, one reading after the timed region"}


ORACLE_BUILD = ("gcc -O3 -march=native -shared -fPIC (the cc backend's command line, arrayjit/lib/cc_backend.ml:77-101) "
                "plus -fno-tree-loop-if-convert (gcc 13.3 miscompiles a vectorised relu gate without it)")


def cpu_baseline(rows, rank=0):
    """The oracle (restated cc backend, one thread as `sync_cc` runs) over the rank's shard of the
    same forward; returns the rate and the loss it computed."""
    from ocannl_b200 import workloads as W
    from oracle.run_c import OracleRoutine
    ir = W.mlp_forward(rows=rows, dims=DIMS)
    o = OracleRoutine(ir.to_b200ir())
    bufs = o.buffers()
    x, onehot = shard_inputs(rows, rank)
    for k, v in dict(W.mlp_params(dims=DIMS), x=x, labels=onehot).items():
        bufs[k][...] = np.asarray(v).reshape(bufs[k].shape)
    t = o.run(bufs)
    return {"value": rows / t, "unit": "samples/s", "cores": 1, "kind": "port", "seconds": round(t, 2),
            "sample": "all %d rows of rank 0's shard, same routine, one run" % rows, "build": ORACLE_BUILD,
            "loss": float(bufs["loss"][0])}


def shard_inputs(rows, rank, total=None):
    """Rows [rank * rows, (rank + 1) * rows) of the one seeded batch (`shard_along`, axis 0)."""
    from ocannl_b200 import workloads as W
    total = total or rows
    x, onehot = W.mlp_inputs(rows=total)
    lo = rank * rows
    return np.ascontiguousarray(x[lo:lo + rows]), np.ascontiguousarray(onehot[lo:lo + rows])


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    from ocannl_b200 import workloads as W
    from oracle.run_c import OracleRoutine
    rows = args.ref_rows
    ir = W.mlp_forward(rows=rows, dims=DIMS)
    o = OracleRoutine(ir.to_b200ir())
    bufs = o.buffers()
    x, onehot = W.mlp_inputs(rows=rows)
    for k, v in dict(W.mlp_params(dims=DIMS), x=x, labels=onehot).items():
        bufs[k][...] = np.asarray(v).reshape(bufs[k].shape)
    for _ in range(max(1, min(args.warmup, 2))):
        o.run(bufs)
    t = sum(o.run(bufs) for _ in range(steps))
    v = rows * steps / t
    sample = "%d rows per step (bounded sample of the %d-row shard), one host thread as the reference's sync_cc" % (
        rows, args.rows)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "samples/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * t / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD % args.rows, "rows_per_step": rows,
                   "rows_per_gpu": args.rows // max(1, args.gpus), "global_batch": args.rows, "parallelism": "dp%d" % args.gpus},
        "cpu_baseline": {"value": v, "unit": "samples/s", "cores": 1, "kind": "port", "sample": sample, "build": ORACLE_BUILD},
        "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def contraction_sweep(dev, pk, sizes=(1024, 4096, 8192)):
    """Config 3: batch 8, M=N=K in {1024, 4096, 8192}, bf16 in, fp32 z + bf16 y out."""
    from ocannl_b200 import backend as bk
    from ocannl_b200 import workloads as W
    out = []
    for n in sizes:
        ir = W.einsum_gelu(8, n, n, n)
        code = bk.Code(ir)
        rt = bk.Context(dev).link(code)
        blk_a = W.store("bfloat16", np.random.default_rng(6).standard_normal((n, n), np.float32))
        blk_b = W.store("bfloat16", np.random.default_rng(7).standard_normal((n, n), np.float32))
        for name, blk in (("a", blk_a), ("b", blk_b)):
            pool, off, t = rt.context.arrays[name]
            for b in range(8):
                dev.from_host(pool, off + b * blk.nbytes, blk)
            dev.await_()
        rt.context.from_host("bias", np.random.default_rng(8).standard_normal(n).astype(np.float32))
        for _ in range(3):
            rt.run()
        dev.await_()
        rt.profile(True)
        reps = 5 if n < 8192 else 3
        for _ in range(reps):
            rt.run()
        dev.await_()
        st = rt.stage_times()
        info = code.info()["stages"]
        gemm_ms = st[0][0] / st[0][1]
        total_ms = sum(t / c for t, c in st if c)
        flops = 2.0 * 8 * n ** 3
        out.append({"n": n, "kernel_ms": gemm_ms, "routine_ms": total_ms, "tflops": flops / gemm_ms / 1e9,
                    "frac_of_bf16_peak": flops / gemm_ms / 1e9 / pk["bf16"], "routine_tflops": flops / total_ms / 1e9,
                    "stages": [s["kind"] for s in info]})
        rt.free()
        code.free()
        for p in {p for p, _, _ in rt.context.arrays.values()}:
            dev.free_pool(p)
    return out


def _time_routine(dev, rt, code, runs, pk, statics=None, flush_pool=None):
    """ms per run with CUDA-graph replay, plus a per-stage breakdown from event-timed runs."""
    statics = statics or [{}]
    rt.use_graph(True)
    for i in range(3):
        rt.run(**statics[i % len(statics)])
    dev.await_()
    total = 0.0
    for i in range(runs):
        if flush_pool is not None:
            dev.memset_zero(flush_pool, 0, 256 << 20)
        e0 = dev.all_work()
        rt.run(**statics[i % len(statics)])
        e1 = dev.all_work()
        e1.sync()
        total += e0.elapsed_ms(e1)
        e0.free()
        e1.free()
    rt.profile(True)
    for i in range(runs):
        if flush_pool is not None:
            for _ in range(4):     # flush L2 and keep the device busy while the host queues stages and events
                dev.memset_zero(flush_pool, 0, 256 << 20)
        rt.run(**statics[i % len(statics)])
    dev.await_()
    rt.profile(False)
    stages = code.info()["stages"]
    out = []
    for s, (t, c) in zip(stages, rt.stage_times()):
        ms = t / c if c else 0.0
        e = {"kernel": s["kernel"] or "memset", "kind": s["kind"], "ms": round(ms, 5), "bytes": s.get("bytes", 0)}
        if ms > 0:
            e["gbs"] = round(s.get("bytes", 0) / ms / 1e6, 1)
            if s["kind"] in ("gemm", "attention"):
                e["tflops"] = round(s["flops"] / ms / 1e9, 1)
        out.append(e)
    return total / runs, out


def other_configs(dev, pk):
    """Configs 1, 2 and 4 of the baseline, each through compile / link / run with graph replay."""
    from ocannl_b200 import backend as bk
    from ocannl_b200 import workloads as W
    res = {}
    flush_pool = dev.alloc_pool(256 << 20)

    def run(ir, inputs, runs, statics=None, flush=True):
        code = bk.Code(ir)
        rt = bk.Context(dev).link(code)
        for k, v in inputs.items():
            rt.context.from_host(k, v)
        ms, stages = _time_routine(dev, rt, code, runs, pk, statics, flush_pool if flush else None)
        n_kernels = rt.kernels_per_run()
        rt.free()
        code.free()
        for p in {p for p, _, _ in rt.context.arrays.values()}:
            dev.free_pool(p)
        return ms, stages, n_kernels

    # launch floor: a routine of one single-thread kernel, replayed as a graph like everything else
    from ocannl_b200.low_level import Routine, Seq, Set
    nop = Routine("launch_floor")
    a_ = nop.tn("a", "single", [1], read_only=True)
    b_ = nop.tn("b", "single", [1])
    nop.body = Seq([Set(b_, (0,), a_[0] + 1.0)])
    floor_ms, _, _ = run(nop, {"a": np.float32([1.0])}, 50, flush=False)
    # config 1: half-moons MLP, one training step per run (batch 20)
    x, y = W.moons_inputs()
    ms, st, nk = run(W.moons_train_step(), dict(W.moons_params(), moons_flat=x, moons_classes=y), 50,
                     [{"i1": i % 51, "i2": i} for i in range(51)], flush=False)
    res["moons_train_step"] = {"ms_per_step": ms, "samples_per_s": 20 / (ms / 1e3), "kernels": nk,
                               "bound": "launch latency", "launch_floor_ms": floor_ms,
                               "floor_fraction": floor_ms / ms if ms else None}
    # config 2: makemore forward, fp32 and bf16 weights
    ids, onehot = W.makemore_inputs()
    for wp in ("single", "bfloat16"):
        inp = {k: W.store(wp, v) for k, v in W.makemore_params().items()}
        inp.update(input_batch=ids, target_batch=onehot)
        ms, st, nk = run(W.makemore_forward(wprec=wp), inp, 30)
        res["makemore_forward_" + wp] = {"ms_per_step": ms, "samples_per_s": 4096 / (ms / 1e3), "kernels": nk,
                                         "stages": st}
    # config 4: decoder-only transformer forward, batch 64 x 256 tokens.  Twice: with the attention
    # chain's intermediate nodes (scores, exponentials, weights: 335 MB per layer) held by the context,
    # so that the fused attention stage must write them, and with those nodes routine-local, where it
    # writes none of them.
    inp = dict(W.transformer_params(), **W.transformer_inputs())
    for key, mode in (("decoder_forward", "ctx"), ("decoder_forward_local_attention_nodes", "local")):
        ir = W.transformer_forward(attn_nodes=mode)
        ms, st, nk = run(ir, inp, 5)
        flops = sum(s_["flops"] for s_ in bk.Code(ir).info()["stages"] if s_["kind"] in ("gemm", "attention"))
        top = sorted(st, key=lambda e: -e["ms"])[:8]
        gen = [e for e in st if e["kind"] == "generic" and e["ms"] > 0]
        att = [e for e in st if e["kind"] == "attention" and e["ms"] > 0]
        res[key] = {
            "ms_per_step": ms, "samples_per_s": 64 / (ms / 1e3), "tokens_per_s": 64 * 256 / (ms / 1e3), "kernels": nk,
            "attention_nodes": "held by the context (written)" if mode == "ctx" else "routine-local (never written)",
            "contraction_tflops_over_whole_step": flops / ms / 1e9, "top_stages": top,
            "generic_stage_time_ms": round(sum(e["ms"] for e in gen), 4),
            "contraction_stage_time_ms": round(sum(e["ms"] for e in st if e["kind"] == "gemm"), 4),
            "attention_stage_time_ms": round(sum(e["ms"] for e in att), 4),
            "attention_stage_gbs": round(sum(e["bytes"] for e in att) / max(sum(e["ms"] for e in att), 1e-9) / 1e6, 1),
            "generic_gbs_weighted": round(sum(e["bytes"] for e in gen) / max(sum(e["ms"] for e in gen), 1e-9) / 1e6, 1),
            "hbm_peak_gbs": pk["hbm"]}
    dev.free_pool(flush_pool)
    return res


def train_step(dev, dist, rank, world, rows, total_rows, K, Wm):
    """Config 5 (ii): per shard forward + backward, one NCCL allreduce (average) over the
    contiguous fp32 gradient range, local SGD on every replica.  Max over ranks of the
    CUDA-event time of K steps."""
    from ocannl_b200 import parallel as par
    from ocannl_b200 import workloads as W
    rep = par.DeviceReplica(dev, W.mlp_train_update(rows=rows, dims=DIMS), W.mlp_sgd(dims=DIMS), W.MLP_PARAM_NAMES)
    if world > 1:
        box = [par.NcclExchange.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ex = par.NcclExchange(dev, world, rank, box[0])
        ex.set_timeout(120000)       # a rank that never arrives ends the wait instead of hanging it
        buckets = ex.attach_overlap(rep, mean=True)
    else:
        ex = par.LocalExchange()
    progress("training step: replica linked, exchange ready")
    h = par.DataParallel(rep, ex, "mean", input_ident="x", target_ident="labels")
    x, onehot = shard_inputs(rows, rank, total_rows)
    rep.set_values(dict(W.mlp_params(dims=DIMS), x=x, labels=onehot, learning_rate=np.float32([0.01])))
    for i in range(Wm):
        h.step()
        if i == 0:
            dev.await_()
            progress("training step: first step done")
    dev.await_()
    progress("training step: warm-up done")
    if dist is not None:
        dist.barrier()
    e0 = dev.all_work()
    for _ in range(K):
        h.step()
    e1 = dev.all_work()
    dev.await_()              # with a communicator timeout this wait polls for NCCL errors instead of blocking
    progress("training step: timed steps done")
    ms = e0.elapsed_ms(e1)
    if dist is not None:
        import torch
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    loss = h.owner_loss_value()
    pool, off, count = rep.grad_range
    kernels = rep.update.kernels_per_run() + rep.sgd.kernels_per_run()
    if world > 1:
        ex.free()
    return {"samples_per_s": rows * world * K / (ms / 1e3), "ms_per_step": ms / K, "allreduce_bytes": int(count) * 4,
            "exchange": ("ncclAllReduce(avg, fp32) in %d buckets on the communicator's stream, each started when its last "
                         "gradient kernel is queued, beside the rest of the backward pass" % len(buckets)) if world > 1 else "none (1 shard)",
            "kernels_per_step": int(kernels), "loss_after": loss}


def probe_attention_scores(dev):
    """The decoder's score contraction as a routine of its own (64 sequences, 256 positions, 8 heads
    of 64), with its mask epilogue, with the scaling only, and bare: what the `where(mask, ..)`
    costs the epilogue.  A small case for profilers and for the numbers quoted beside the kernel."""
    import math
    from ocannl_b200 import backend as bk
    from ocannl_b200 import workloads as W
    from ocannl_b200.low_level import Const, Routine, Seq, Set, loops, where
    B, S, H, E = 64, 256, 8, 64
    out = {}
    for variant in ("mask", "scale", "bare"):
        r = Routine("scores_" + variant)
        q = r.tn("q", "bfloat16", [B, S, H, E], read_only=True)
        k = r.tn("k", "bfloat16", [B, S, H, E], read_only=True)
        mask = r.tn("mask", "single", [S, S], read_only=True)
        scores = r.tn("scores", "single", [B, S, H, S])
        b, s_, h, t, e = r.syms(5)
        acc = W.reduce_scope(r, "qk", "single", [(e, E)], lambda: (q[b, s_, h, e], k[b, t, h, e]), orig=(b, s_, h, t))
        val = where(mask[s_, t], acc / math.sqrt(E), Const(-1e9)) if variant == "mask" else (acc / math.sqrt(E) if variant == "scale" else acc)
        r.body = Seq([loops([(b, B), (s_, S), (h, H), (t, S)], Set(scores, (b, s_, h, t), val))])
        code = bk.Code(r)
        rt = bk.Context(dev).link(code)
        g = np.random.default_rng(0)
        rt.context.from_host("q", W.store("bfloat16", g.standard_normal((B, S, H, E), np.float32)))
        rt.context.from_host("k", W.store("bfloat16", g.standard_normal((B, S, H, E), np.float32)))
        if variant == "mask":
            rt.context.from_host("mask", (np.arange(S)[:, None] >= np.arange(S)[None, :]).astype(np.float32))
        for _ in range(3):
            rt.run()
        dev.await_()
        e0 = dev.all_work()
        for _ in range(10):
            rt.run()
        e1 = dev.all_work()
        e1.sync()
        ms = e0.elapsed_ms(e1) / 10
        nbytes = 2 * B * S * H * E * 2 + B * S * H * S * 4
        out[variant] = {"us": round(1e3 * ms, 2), "gbs": round(nbytes / ms / 1e6, 1), "note": rt.info()["stages"][0]["note"]}
        pools = {p for p, _, _ in rt.context.arrays.values()}
        rt.free()
        code.free()
        for p in pools:
            dev.free_pool(p)
    return out


def probe_attention(dev, batch=64, heads=8, seq=256):
    """One attention layer of the decoder as a routine of its own (64 sequences, 256 positions, 8
    heads of 64): the fused stage with the intermediate nodes held by the context (all written) and
    routine-local (none written), and the separate stages (`attn=0`).  A small case for profilers and
    for the numbers quoted beside the kernel."""
    from ocannl_b200 import backend as bk
    from ocannl_b200 import workloads as W
    out = {}
    inputs = W.attention_inputs(batch, heads, seq, seq)
    for key, mode, options in (("fused, nodes kept", "ctx", None), ("fused, nodes local", "local", None),
                               ("separate stages, nodes kept", "ctx", "attn=0")):
        code = bk.Code(W.attention(batch, heads, seq, seq, row_mode=mode), options)
        rt = bk.Context(dev).link(code)
        for k, v in inputs.items():
            rt.context.from_host(k, v)
        for _ in range(3):
            rt.run()
        dev.await_()
        e0 = dev.all_work()
        for _ in range(10):
            rt.run()
        e1 = dev.all_work()
        e1.sync()
        ms = e0.elapsed_ms(e1) / 10
        st = rt.info()["stages"]
        out[key] = {"us": round(1e3 * ms, 2), "kernels": rt.kernels_per_run(), "bytes": sum(s_["bytes"] for s_ in st),
                    "gbs": round(sum(s_["bytes"] for s_ in st) / ms / 1e6, 1), "notes": [s_["note"] for s_ in st]}
        pools = {p for p, _, _ in rt.context.arrays.values()}
        rt.free()
        code.free()
        for p in pools:
            dev.free_pool(p)
    return out


def probe_ffn(dev, batch=64, seq=256, d_model=512, d_ff=2048):
    """The first feed-forward contraction of a decoder layer as a routine of its own: 16384 rows,
    K = 512, N = 2048, bias, the pre-activation kept in single precision and the composed GELU
    written as bfloat16 -- a contraction whose epilogue outweighs its main loop.  A small case for
    profilers."""
    from ocannl_b200 import backend as bk
    from ocannl_b200 import workloads as W
    from ocannl_b200.low_level import Routine, Seq, Set, loops
    r = Routine("ffn_in_b%d_s%d" % (batch, seq))
    x = r.tn("x", "bfloat16", [batch, seq, d_model], read_only=True)
    w = r.tn("w", "bfloat16", [d_ff, d_model], read_only=True)
    bias = r.tn("b", "bfloat16", [d_ff], read_only=True)
    z = r.tn("z", "single", [batch, seq, d_ff])
    h = r.tn("h", "bfloat16", [batch, seq, d_ff])
    b, s_, j, i = r.syms(4)
    pre = W.reduce_scope(r, "n_ffn", "single", [(i, d_model)], lambda: (w[j, i], x[b, s_, i]), orig=(b, s_, j)) + bias[j]
    b2, s2, j2 = r.syms(3)
    r.body = Seq([loops([(b, batch), (s_, seq), (j, d_ff)], Set(z, (b, s_, j), pre)),
                  loops([(b2, batch), (s2, seq), (j2, d_ff)], Set(h, (b2, s2, j2), W.gelu_tanh(z[b2, s2, j2])))])
    code = bk.Code(r)
    rt = bk.Context(dev).link(code)
    g = np.random.default_rng(0)
    rt.context.from_host("x", W.store("bfloat16", g.standard_normal((batch, seq, d_model), np.float32)))
    rt.context.from_host("w", W.store("bfloat16", (g.standard_normal((d_ff, d_model), np.float32) / np.sqrt(d_model)).astype(np.float32)))
    rt.context.from_host("b", W.store("bfloat16", g.standard_normal((d_ff,), np.float32)))
    for _ in range(3):
        rt.run()
    dev.await_()
    e0 = dev.all_work()
    for _ in range(10):
        rt.run()
    e1 = dev.all_work()
    e1.sync()
    ms = e0.elapsed_ms(e1) / 10
    st = rt.info()["stages"]
    flops = 2.0 * batch * seq * d_model * d_ff
    out = {"us": round(1e3 * ms, 2), "kernels": rt.kernels_per_run(), "tflops": round(flops / ms / 1e9, 1),
           "bytes": sum(s_["bytes"] for s_ in st), "gbs": round(sum(s_["bytes"] for s_ in st) / ms / 1e6, 1),
           "notes": [s_["note"] for s_ in st]}
    pools = {p for p, _, _ in rt.context.arrays.values()}
    rt.free()
    code.free()
    for p in pools:
        dev.free_pool(p)
    return out


def probe_layer_norm(dev, batch=64, seq=256, d_model=512, eps=1e-5):
    """One layer norm of the decoder as a routine of its own (`layer_norm`, lib/nn_blocks.ml:251-258, on
    16384 rows of 512 bf16 features: row sum, centring, root of the summed squares, scale and shift).
    A small case for profilers."""
    from ocannl_b200 import backend as bk
    from ocannl_b200 import workloads as W
    from ocannl_b200.low_level import Routine, Seq, Set, loops, un
    r = Routine("layer_norm_b%d_s%d" % (batch, seq))
    B, S, D = batch, seq, d_model
    src = r.tn("x", "bfloat16", [B, S, D], read_only=True)
    out = r.tn("y", "bfloat16", [B, S, D])
    ssum = r.tn("sum", "single", [B, S, 1])
    cen = r.tn("centered", "single", [B, S, D])
    std = r.tn("std", "single", [B, S, 1])
    gamma = r.tn("gamma", "single", [D], read_only=True)
    beta = r.tn("beta", "single", [D], read_only=True)
    body = []
    b, s_, d = r.syms(3)
    body.append(loops([(b, B), (s_, S)], Set(ssum, (b, s_, 0), W.reduce_scope(r, "n_sum", "single", [(d, D)], lambda: src[b, s_, d], op="add"))))
    b, s_, d = r.syms(3)
    body.append(loops([(b, B), (s_, S), (d, D)], Set(cen, (b, s_, d), (src[b, s_, d] - ssum[b, s_, 0]) / float(D))))
    b, s_, d = r.syms(3)
    body.append(loops([(b, B), (s_, S)], Set(std, (b, s_, 0), un("sqrt", W.reduce_scope(
        r, "n_var", "single", [(d, D)], lambda: cen[b, s_, d] * cen[b, s_, d], op="add") + eps))))
    b, s_, d = r.syms(3)
    body.append(loops([(b, B), (s_, S), (d, D)], Set(out, (b, s_, d), (gamma[d] * (cen[b, s_, d] / std[b, s_, 0])) + beta[d])))
    r.body = Seq(body)
    code = bk.Code(r)
    rt = bk.Context(dev).link(code)
    g = np.random.default_rng(0)
    rt.context.from_host("x", W.store("bfloat16", g.standard_normal((B, S, D), np.float32)))
    rt.context.from_host("gamma", np.ones(D, np.float32))
    rt.context.from_host("beta", np.zeros(D, np.float32))
    for _ in range(3):
        rt.run()
    dev.await_()
    e0 = dev.all_work()
    for _ in range(10):
        rt.run()
    e1 = dev.all_work()
    e1.sync()
    ms = e0.elapsed_ms(e1) / 10
    st = rt.info()["stages"]
    nbytes = sum(s_i["bytes"] for s_i in st)
    out_ = {"us": round(1e3 * ms, 2), "kernels": rt.kernels_per_run(), "bytes": nbytes, "gbs": round(nbytes / ms / 1e6, 1),
            "notes": [s_i["note"] for s_i in st]}
    pools = {p for p, _, _ in rt.context.arrays.values()}
    rt.free()
    code.free()
    for p in pools:
        dev.free_pool(p)
    return out_


def oracle_rate(ir, inputs, units, statics=None, what=""):
    """Seconds of one oracle run of `ir` (one host thread) -> units per second, with the sample stated."""
    from oracle.run_c import OracleRoutine
    o = OracleRoutine(ir.to_b200ir())
    bufs = o.buffers()
    for k, v in inputs.items():
        bufs[k][...] = np.asarray(v).reshape(bufs[k].shape)
    t = o.run(bufs, statics or {})
    return {"value": units / t, "cores": 1, "kind": "port", "seconds": round(t, 3), "sample": what}


def config_cpu_baselines():
    """The oracle beside configs 1-4: one host core, bounded samples (stated per entry)."""
    from ocannl_b200 import workloads as W
    out = {}
    x, y = W.moons_inputs()
    out["moons_train_step"] = dict(oracle_rate(W.moons_train_step(), dict(W.moons_params(), moons_flat=x, moons_classes=y), 20,
                                               {"i1": 0, "i2": 0}, "one training step, batch 20"), unit="samples/s")
    ids, onehot = W.makemore_inputs()
    for wp in ("single", "bfloat16"):
        inp = {k: W.store(wp, v) for k, v in W.makemore_params().items()}
        inp.update(input_batch=ids, target_batch=onehot)
        out["makemore_forward_" + wp] = dict(oracle_rate(W.makemore_forward(wprec=wp), inp, 4096, None, "the whole 4096-row batch"),
                                             unit="samples/s")
    r = oracle_rate(W.einsum_gelu(1, 1024, 1024, 1024), W.einsum_gelu_inputs(1, 1024, 1024, 1024), 2.0 * 1024 ** 3 / 1e9, None,
                    "one of the 8 batch entries at M=N=K=1024 (the entries are independent: the rate carries over)")
    out["einsum_gelu_1024"] = dict(r, unit="GFLOP/s")
    r = oracle_rate(W.transformer_forward(batch=1), dict(W.transformer_params(), **W.transformer_inputs(batch=1)), 256, None,
                    "one sequence of 256 tokens at full width (6 layers, d_model 512); the batch of 64 repeats it")
    out["decoder_forward"] = dict(r, unit="tokens/s")
    return out


def measure_forward(dev, dist, rank, world, rows, total_rows, K, Wm, pk, e2e=True, stages=True, clock_index=None):
    """Times the forward over this rank's `rows`-row shard of the `total_rows`-row batch: device
    resident (per-step CUDA events, L2 flushed between steps), end to end through
    from_host / run / to_host, and per stage.  Returns a dict; times are the max over ranks."""
    from ocannl_b200 import backend as bk
    from ocannl_b200 import workloads as W
    ir = W.mlp_forward(rows=rows, dims=DIMS)
    code = bk.Code(ir)
    rt = bk.Context(dev).link(code)
    ctx = rt.context
    params = W.mlp_params(dims=DIMS)
    x, onehot = shard_inputs(rows, rank if total_rows > rows else 0, total_rows)
    for k, v in params.items():
        ctx.from_host(k, v)
    ctx.from_host("x", x)
    ctx.from_host("labels", onehot)
    flush_pool = dev.alloc_pool(256 << 20)
    rt.use_graph(True)
    res = {"rows": rows, "kernels_per_step": int(rt.kernels_per_run())}

    def barrier():
        dev.await_()
        if dist is not None:
            dist.barrier()

    def timed(step_fn, n):
        total = 0.0
        for _ in range(n):
            dev.memset_zero(flush_pool, 0, 256 << 20)      # L2 flush, outside the events
            e0 = dev.all_work()
            step_fn()
            e1 = dev.all_work()
            e1.sync()
            total += e0.elapsed_ms(e1)
            e0.free()
            e1.free()
        return total

    def max_over_ranks(ms):
        if dist is None:
            return ms
        import torch
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    sampler = ClockSampler(clock_index) if clock_index is not None else None
    if sampler:
        sampler.start()          # runs through warm-up, the timed steps and the end-to-end steps
    for _ in range(Wm):
        rt.run()
    barrier()
    ms = timed(rt.run, K)
    barrier()
    res["ms"] = max_over_ranks(ms)
    progress("  resident forward timed")

    if e2e:
        # host batch in, loss out, through from_host / run / to_host.  The batch of step i + 1 is
        # uploaded (second stream, second input buffer) while step i computes; every step's upload
        # and loss read-back lie inside the timed region, which spans all K steps.
        hx = bk.PinnedBuffer(x.shape, x.dtype)
        hl = bk.PinnedBuffer(onehot.shape, onehot.dtype)
        hloss = [bk.PinnedBuffer((1,), np.float32), bk.PinnedBuffer((1,), np.float32)]
        hx.array[...] = x
        hl.array[...] = onehot
        dev.set_async_uploads(True)
        rt2 = bk.Context(dev).link(code)
        for k, v in params.items():
            rt2.context.from_host(k, v)
        rt2.use_graph(True)
        rts = [rt, rt2]
        slots = [(r.context.arrays["x"], r.context.arrays["labels"], r.context.arrays["loss"]) for r in rts]

        def upload(i):
            (px, ox, _), (pl, ol, _), _ = slots[i % 2]
            dev.from_host(px, ox, hx.array)
            dev.from_host(pl, ol, hl.array)

        def e2e_steps(n):
            upload(0)
            for i in range(n):
                if i + 1 < n:
                    upload(i + 1)
                dev.memset_zero(flush_pool, 0, 256 << 20)      # L2 flush between steps, beside the next upload
                rts[i % 2].run()
                ps, os_, _ = slots[i % 2][2]
                dev.to_host(ps, os_, hloss[i % 2].array)

        e2e_steps(Wm)
        barrier()
        e0 = dev.all_work()
        e2e_steps(K)
        e1 = dev.all_work()
        e1.sync()
        ms_e2e = e0.elapsed_ms(e1)
        e0.free()
        e1.free()
        barrier()
        res["ms_e2e"] = max_over_ranks(ms_e2e)
        progress("  end-to-end forward timed")
        dev.set_async_uploads(False)
        res["loss"] = float(hloss[(K - 1) % 2].array[0])
        res["h2d_bytes"] = int(x.nbytes + onehot.nbytes)
        for b in [hx, hl] + hloss:
            b.free()
        rt2.free()
    if sampler:
        res["clocks"] = sampler.stop()

    if stages:
        # per stage, with CUDA events around every stage (an event pair adds 2-4 us to what it
        # brackets: good for shares and for the long kernels, too high for the short ones)
        rt.profile(True)
        for _ in range(K):
            # several clears: they flush L2 and keep the device busy while the host queues the stages
            # and their events, so that an event pair brackets device time, not the host's launch calls
            for _ in range(4):
                dev.memset_zero(flush_pool, 0, 256 << 20)
            rt.run()
        dev.await_()
        st = rt.stage_times()
        info = rt.info()["stages"]
        res["stage_ms"] = [round(t / c if c else 0.0, 5) for t, c in st]
        res["stage_info"] = info
        rt.profile(False)
    rt.free()
    code.free()
    dev.free_pool(flush_pool)
    return res


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the hidden-layer
# contraction kernels, from the `ncu --set full` capture of these kernels at these shapes that
# the profile summaries of this repository describe.  Not measured in the run: a profiler cannot
# run inside a timed benchmark.  Keyed by (m, n, k); dropped when the kernel's tiling changes.
NCU_TRAFFIC = {(8192, 1024, 784): 14483456, (8192, 1024, 1024): 18906880}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--rows", type=int, default=8192, help="rows of the one batch that is split over the GPUs")
    ap.add_argument("--ref-rows", type=int, default=512)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-train", action="store_true", help="skip the forward+backward+allreduce+SGD section")
    ap.add_argument("--no-configs", action="store_true", help="skip the configs 1, 2 and 4 section")
    ap.add_argument("--sweep-size", type=int, default=0,
                    help="run only the batch-8 contraction of this M=N=K (a small case for profilers) and exit")
    ap.add_argument("--probe", default="", help="'attention_scores': time the decoder's score contraction alone and exit; "
                    "'attention' / 'attention_small': one attention layer alone (64 x 8 or 8 x 8 (batch, head) pairs); "
                    "'ffn': a decoder layer's first feed-forward contraction alone; 'layer_norm': one layer norm alone")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo")
        if _NCCL_VERSION_WANTED and rank == 0:
            import torch
            print("NCCL version %s" % (".".join(str(v) for v in torch.cuda.nccl.version()),), file=sys.stderr)

    from ocannl_b200 import backend as bk
    if not os.path.exists(bk.LIB_PATH):
        from ocannl_b200 import build
        build.build_library()
    pk = peaks()
    dev = bk.Device(local)
    if args.sweep_size:
        print(json.dumps({"contraction_sweep": contraction_sweep(dev, pk, (args.sweep_size,))}))
        return
    if args.probe in ("attention", "attention_small"):
        print(json.dumps({args.probe: probe_attention(dev, batch=64 if args.probe == "attention" else 8)}))
        return
    if args.probe == "layer_norm":
        print(json.dumps({"layer_norm": probe_layer_norm(dev)}))
        return
    if args.probe == "ffn":
        print(json.dumps({"ffn": probe_ffn(dev)}))
        return
    if args.probe == "attention_scores":
        print(json.dumps({"attention_scores": probe_attention_scores(dev)}))
        return
    total_rows, K, Wm = args.rows, max(1, args.steps), max(3, args.warmup)
    if total_rows % world != 0:
        raise SystemExit("--rows must be divisible by the number of GPUs (shard_along splits evenly)")
    rows = total_rows // world

    # ---- the stated workload: one batch split over the ranks
    progress("forward, %d rows per GPU" % rows)
    fwd = measure_forward(dev, dist, rank, world, rows, total_rows, K, Wm, pk, clock_index=local if rank == 0 else None)
    value = total_rows * K / (fwd["ms"] / 1e3)
    # ---- weak scaling beside it: every GPU keeps all the rows (N = 1: the same measurement)
    weak = None
    if world > 1:
        progress("forward, weak scaling: %d rows per GPU" % total_rows)
        w = measure_forward(dev, dist, rank, world, total_rows, total_rows, K, Wm, pk, e2e=False, stages=False)
        weak = {"rows_per_gpu": total_rows, "value": total_rows * world * K / (w["ms"] / 1e3), "unit": "samples/s",
                "ms_per_step": w["ms"] / K}

    # ---- roofline of the dominant kernel
    stages, shares = fwd["stage_info"], fwd["stage_ms"]
    gemm_idx = [i for i, s_ in enumerate(stages) if s_["kind"] == "gemm"]
    # the dominant kernel: the longest contraction stage; stages within 5 % of it (the two hidden layers
    # trade places from run to run) are told apart by their algorithmic work, so that the line names the
    # same kernel every time
    longest = max(shares[i] for i in gemm_idx)
    dom = max((i for i in gemm_idx if shares[i] >= 0.95 * longest), key=lambda i: stages[i]["flops"])
    dom_ms = shares[dom]
    achieved = stages[dom]["flops"] / dom_ms / 1e9
    shape = {k: stages[dom][k] for k in ("m", "n", "k", "batch")}
    roofline = {"bound": "tensor", "achieved": achieved, "peak": pk["bf16"], "unit": "TFLOP/s",
                "frac": achieved / pk["bf16"], "traffic": None, "peak_source": pk["source"] + " (burst)",
                "kernel": stages[dom]["kernel"], "kernel_ms": dom_ms, "shape": shape, "stage_ms": shares,
                "stage_ms_note": "per-stage CUDA event pairs; each pair adds 2-4 us to its stage, so the sum exceeds ms_per_step",
                "whole_step_frac": sum(stages[i]["flops"] for i in gemm_idx) / (fwd["ms"] / K) / 1e9 / pk["bf16"]}
    key = (shape["m"], shape["n"], shape["k"])
    if key in NCU_TRAFFIC and "CTA pair" in (stages[dom]["note"] or ""):
        roofline["traffic"] = NCU_TRAFFIC[key]
        roofline["traffic_source"] = ("ncu --set full capture of this kernel at this shape, bytes per launch with a cold L2 "
                                      "(outputs stay in L2); from an earlier capture, not measured in this run")
        roofline["algorithmic_bytes"] = stages[dom]["bytes"]

    train = None
    if not args.no_train:
        progress("training step")
        train = train_step(dev, dist, rank, world, rows, total_rows, K, Wm)

    progress("measurements done")
    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": Wm,
        "ms_per_step": fwd["ms"] / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD % total_rows,
                   "rows_per_gpu": rows, "global_batch": total_rows, "parallelism": "dp%d" % world,
                   "l2": "flushed between steps (256 MiB clear outside the per-step CUDA events)",
                   "launch": "CUDA graph replay of the routine's stages"},
        "e2e": {"value": total_rows * K / (fwd["ms_e2e"] / 1e3), "unit": "samples/s",
                "h2d_bytes_per_step": fwd["h2d_bytes"], "d2h_bytes_per_step": 4,
                "ms_per_step": fwd["ms_e2e"] / K,
                "pipeline": "upload of batch i+1 (second stream, second input buffer) overlaps step i; one timed "
                            "region over all steps; L2 cleared before every step"},
        "gpu_launches": fwd["kernels_per_step"] * K,
        "clocks": fwd.get("clocks"), "roofline": roofline, "loss": fwd["loss"],
    }
    if weak is not None:
        line["weak"] = weak
    if train is not None:
        line["train_step"] = train
    if not args.no_cpu:
        cb = cpu_baseline(rows, 0)
        line["cpu_baseline"] = cb
        rel = abs(cb["loss"] - fwd["loss"]) / max(abs(cb["loss"]), 1e-30)
        line["loss_check"] = {"oracle": cb["loss"], "device": fwd["loss"], "rel_err": rel, "tolerance": 1e-3}
        if not rel <= 1e-3:
            raise SystemExit("the device's loss %r differs from the oracle's %r" % (fwd["loss"], cb["loss"]))
    if world == 1 and not args.no_sweep:
        sweep = contraction_sweep(dev, pk)
        roofline["contraction"] = {str(e["n"]): {"ms": round(e["kernel_ms"], 4), "tflops": round(e["tflops"], 1),
                                                 "frac": round(e["frac_of_bf16_peak"], 3)} for e in sweep}
    if world == 1 and not args.no_configs:
        line["configs"] = other_configs(dev, pk)
        if not args.no_cpu:
            for k, v in config_cpu_baselines().items():
                if k in line["configs"]:
                    line["configs"][k]["cpu_baseline"] = v
                else:
                    line["configs"][k] = {"cpu_baseline": v}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
