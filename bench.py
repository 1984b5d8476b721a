"""Benchmark of the hot path: batch-sharded inference forward of the 784-1024-1024-10 MLP.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One process per GPU (the launcher is torch.distributed.run for N > 1); every rank runs the
forward routine over its own shard of `--rows` rows (weak scaling, no data-path collective —
inference forward shards by batch).  A step = one run of the routine over one batch.

Reported on ONE JSON line by rank 0:
  value      forward samples/s of the whole job, inputs resident in device memory
  e2e        the same through the host-facing calls: page-locked host batch -> from_host ->
             run -> to_host of the loss, copies inside the timed region
  roofline   the dominant kernel (the widest hidden-layer contraction): algorithmic FLOPs /
             its CUDA-event duration, against the measured bf16 peak
  cpu_baseline  the restated cc backend (oracle) on one host core, on a bounded row sample
  contraction_sweep  `b|m,k ; b|k,n => b|m,n` + bias + GELU at 1024/4096/8192, TFLOP/s and
             fraction of the measured bf16 peak (rank 0, N = 1 only)
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
DIMS = (784, 1024, 1024, 10)


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


def cpu_baseline(target_s=12.0):
    """The oracle (restated cc backend, gcc -O3 -march=native, one thread as `sync_cc` runs)
    on a row sample of the same forward; returns samples/s."""
    from ocannl_b200 import workloads as W
    from oracle.run_c import OracleRoutine

    def run(rows):
        ir = W.mlp_forward(rows=rows, dims=DIMS)
        o = OracleRoutine(ir.to_b200ir())
        bufs = o.buffers()
        x, onehot = W.mlp_inputs(rows=rows)
        for k, v in dict(W.mlp_params(dims=DIMS), x=x, labels=onehot).items():
            bufs[k][...] = np.asarray(v).reshape(bufs[k].shape)
        o.run(bufs)                       # warm-up
        ts = [o.run(bufs) for _ in range(3)]
        return float(np.median(ts))

    t = run(64)
    rows = int(min(8192, max(64, 64 * target_s / (4 * max(t, 1e-6)))))
    rows = max(64, rows // 64 * 64)
    t = run(rows)
    return {"value": rows / t, "unit": "samples/s", "cores": 1, "kind": "port",
            "sample": "%d of the shard's rows, same routine, median of 3 runs after 1 warm-up" % rows}


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
        "warmup": args.warmup, "ms_per_step": 1e3 * t / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "config 5 forward: MLP 784-1024-1024-10, bf16 weights, fp32 accumulation, softmax CE",
                   "rows_per_step": rows},
        "cpu_baseline": {"value": v, "unit": "samples/s", "cores": 1, "kind": "port", "sample": sample},
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
            if s["kind"] == "gemm":
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
    # config 4: decoder-only transformer forward, batch 64 x 256 tokens
    ir = W.transformer_forward()
    inp = dict(W.transformer_params(), **W.transformer_inputs())
    ms, st, nk = run(ir, inp, 5)
    flops = sum(s_["flops"] for s_ in bk.Code(ir).info()["stages"] if s_["kind"] == "gemm")
    top = sorted(st, key=lambda e: -e["ms"])[:8]
    gen = [e for e in st if e["kind"] == "generic" and e["ms"] > 0]
    res["decoder_forward"] = {
        "ms_per_step": ms, "samples_per_s": 64 / (ms / 1e3), "tokens_per_s": 64 * 256 / (ms / 1e3), "kernels": nk,
        "contraction_tflops_over_whole_step": flops / ms / 1e9, "top_stages": top,
        "generic_stage_time_ms": round(sum(e["ms"] for e in gen), 4),
        "contraction_stage_time_ms": round(sum(e["ms"] for e in st if e["kind"] == "gemm"), 4),
        "generic_gbs_weighted": round(sum(e["bytes"] for e in gen) / max(sum(e["ms"] for e in gen), 1e-9) / 1e6, 1),
        "hbm_peak_gbs": pk["hbm"]}
    dev.free_pool(flush_pool)
    return res


def train_step(dev, dist, rank, world, rows, K, Wm):
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
    else:
        ex = par.LocalExchange()
    h = par.DataParallel(rep, ex, "mean", input_ident="x", target_ident="labels")
    x, onehot = W.mlp_inputs(rows=rows, seed=20 + rank, label_seed=21 + rank)
    rep.set_values(dict(W.mlp_params(dims=DIMS), x=x, labels=onehot, learning_rate=np.float32([0.01])))
    for _ in range(Wm):
        h.step()
    dev.await_()
    if dist is not None:
        dist.barrier()
    e0 = dev.all_work()
    for _ in range(K):
        h.step()
    e1 = dev.all_work()
    e1.sync()
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
            "exchange": "ncclAllReduce(avg, fp32) over one contiguous gradient range" if world > 1 else "none (1 shard)",
            "kernels_per_step": int(kernels), "loss_after": loss}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--rows", type=int, default=8192, help="rows of the batch each GPU processes per step")
    ap.add_argument("--ref-rows", type=int, default=512)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-train", action="store_true", help="skip the forward+backward+allreduce+SGD section")
    ap.add_argument("--no-configs", action="store_true", help="skip the configs 1, 2 and 4 section")
    ap.add_argument("--sweep-size", type=int, default=0,
                    help="run only the batch-8 contraction of this M=N=K (a small case for profilers) and exit")
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

    # run this rank on the host cores next to its GPU, so that its page-locked batches are
    # allocated in that socket's memory (a property of this process, not of the GPU)
    numa = None
    if world > 1:
        try:
            import pynvml
            pynvml.nvmlInit()
            pynvml.nvmlDeviceSetCpuAffinity(pynvml.nvmlDeviceGetHandleByIndex(local))
            numa = "cpu affinity of the rank set to its GPU's cores (NVML)"
        except Exception as e:      # not fatal: the copies then may cross sockets
            numa = "cpu affinity not set: %s" % (e,)

    from ocannl_b200 import backend as bk
    from ocannl_b200 import workloads as W
    if not os.path.exists(bk.LIB_PATH):
        from ocannl_b200 import build
        build.build_library()
    pk = peaks()
    dev = bk.Device(local)
    if args.sweep_size:
        print(json.dumps({"contraction_sweep": contraction_sweep(dev, pk, (args.sweep_size,))}))
        return
    rows, K, Wm = args.rows, max(1, args.steps), max(3, args.warmup)
    ir = W.mlp_forward(rows=rows, dims=DIMS)
    code = bk.Code(ir)
    rt = bk.Context(dev).link(code)
    ctx = rt.context
    # every rank holds the same parameters and its own shard of rows (seeded by rank)
    params = W.mlp_params(dims=DIMS)
    x, onehot = W.mlp_inputs(rows=rows, seed=20 + rank, label_seed=21 + rank)
    for k, v in params.items():
        ctx.from_host(k, v)
    ctx.from_host("x", x)
    ctx.from_host("labels", onehot)
    flush_pool = dev.alloc_pool(256 << 20)
    rt.use_graph(True)

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

    # ---- device-resident forward
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()          # runs through warm-up, the timed steps and the end-to-end steps
    for _ in range(Wm):
        rt.run()
    barrier()
    ms = timed(rt.run, K)
    barrier()
    ms = max_over_ranks(ms)
    value = rows * world * K / (ms / 1e3)

    # ---- end to end: host batch in, loss out, through from_host / run / to_host.  The batch of
    # step i + 1 is uploaded (second stream, second input buffer) while step i computes; every
    # step's upload and loss read-back lie inside the timed region, which spans all K steps.
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
    ms_e2e = max_over_ranks(ms_e2e)
    dev.set_async_uploads(False)
    loss_value = float(hloss[(K - 1) % 2].array[0])
    clocks = sampler.stop() if rank == 0 else None

    # ---- roofline of the dominant kernel, timed per stage with CUDA events
    rt.profile(True)
    for _ in range(K):
        # several clears: they flush L2 and keep the device busy while the host queues the stages
        # and their events, so that an event pair brackets device time, not the host's launch calls
        for _ in range(4):
            dev.memset_zero(flush_pool, 0, 256 << 20)
        rt.run()
    dev.await_()
    st = rt.stage_times()
    stages = code.info()["stages"]
    shares = [(t / c if c else 0.0) for t, c in st]
    dom = max((i for i, s in enumerate(stages) if s["kind"] == "gemm"), key=lambda i: shares[i])
    dom_ms = shares[dom]
    achieved = stages[dom]["flops"] / dom_ms / 1e9
    roofline = {"bound": "tensor", "achieved": achieved, "peak": pk["bf16"], "unit": "TFLOP/s",
                "frac": achieved / pk["bf16"], "traffic": None, "peak_source": pk["source"] + " (burst)",
                "kernel": stages[dom]["kernel"], "kernel_ms": dom_ms,
                "shape": {k: stages[dom][k] for k in ("m", "n", "k", "batch")},
                "stage_ms": [round(s, 5) for s in shares]}
    # DRAM bytes of one launch from the ncu capture summarised in
    # profiles/contraction_mlp_layer_8192x1024x784.md (dram__bytes_read.sum + dram__bytes_write.sum)
    ncu_traffic = {"mlp_fwd_8192_s0": 14483456, "mlp_fwd_8192_s1": 18906880}
    if stages[dom]["kernel"] in ncu_traffic:
        roofline["traffic"] = ncu_traffic[stages[dom]["kernel"]]
        roofline["traffic_unit"] = "bytes per launch (ncu, cold L2; outputs stay in L2)"
        roofline["algorithmic_bytes"] = stages[dom]["bytes"]
    rt.profile(False)

    train = None if args.no_train else train_step(dev, dist, rank, world, rows, K, Wm)

    if rank != 0:
        return
    line = {
        "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": Wm,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "config 5 forward: MLP 784-1024-1024-10, bf16 weights and activations, fp32 "
                               "accumulation, softmax cross-entropy; batch-sharded, no collective",
                   "rows_per_gpu": rows, "global_batch": rows * world, "parallelism": "dp%d" % world,
                   "l2": "flushed between steps (256 MiB clear outside the per-step CUDA events)",
                   "launch": "CUDA graph replay of the routine's stages", "host_placement": numa},
        "e2e": {"value": rows * world * K / (ms_e2e / 1e3), "unit": "samples/s",
                "h2d_bytes_per_step": int(x.nbytes + onehot.nbytes), "d2h_bytes_per_step": 4,
                "ms_per_step": ms_e2e / K,
                "pipeline": "upload of batch i+1 (second stream, second input buffer) overlaps step i; one timed "
                            "region over all steps; L2 cleared before every step"},
        "gpu_launches": int(rt.kernels_per_run()) * K,
        "clocks": clocks, "roofline": roofline, "loss": loss_value,
    }
    if train is not None:
        line["train_step"] = train
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline()
    if world == 1 and not args.no_sweep:
        line["contraction_sweep"] = contraction_sweep(dev, pk)
    if world == 1 and not args.no_configs:
        line["configs"] = other_configs(dev, pk)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
