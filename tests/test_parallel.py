"""Data-parallel driver: sharding helpers, the reference's known answers for a 1-shard and a
2-shard step (test/training/data_parallel.expected: losses 67.5 / 11.25, w = 5.0 both ways),
over gloo ranks on CPU (replicas run the CPU oracle) and over NCCL on two GPUs."""
import os
import sys

import numpy as np
import pytest
import torch  # noqa: F401  (before anything opens libnccl: the loader reuses an already loaded libnccl.so.2 for
              # torch's own dependency, and the system's copy may be older than the one torch was built against)

from ocannl_b200 import parallel as par
from ocannl_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
X = np.float32([[1.], [2.], [3.], [4.]])
Y = np.float32([[2.], [4.], [6.], [8.]])


def test_shard_and_gather_round_trip():
    a = np.arange(24, dtype=np.float32).reshape(6, 4)
    sh = par.shard_along(a, 3)
    assert [s.shape for s in sh] == [(2, 4)] * 3 and np.array_equal(sh[1], a[2:4])
    assert np.array_equal(par.gather(sh), a)
    for bad in (lambda: par.shard_along(a, 4), lambda: par.shard_along(a, 0), lambda: par.shard_along(a, 2, axis=1),
                lambda: par.shard_along(np.float32(1.0), 1), lambda: par.gather([]),
                lambda: par.gather([a, a[:, :2]])):
        with pytest.raises(ValueError):
            bad()


class OracleReplica:
    """Stand-in replica for CPU ranks: the routines run through the CPU oracle."""

    def __init__(self, update_ir, sgd_ir, params, loss="loss"):
        from oracle.run_c import OracleRoutine
        self.update, self.sgd = OracleRoutine(update_ir.to_b200ir()), OracleRoutine(sgd_ir.to_b200ir())
        self.bufs = self.update.buffers()
        for k, v in self.sgd.buffers().items():
            self.bufs.setdefault(k, v)
        self.params, self.loss_ident = list(params), loss
        self.grads = [p + "_grad" for p in params]

    def set_values(self, values):
        for k, v in values.items():
            self.bufs[k][...] = np.asarray(v).reshape(self.bufs[k].shape)

    def forward_backward(self, **static):
        self.update.run(self.bufs, static)

    def optimizer_step(self, **static):
        self.sgd.run(self.bufs, static)

    def read(self, ident):
        return self.bufs[ident].copy()

    def await_(self):
        pass


class GlooExchange:
    def __init__(self, dist):
        self.dist, self.n_ranks, self.rank = dist, dist.get_world_size(), dist.get_rank()

    def allreduce(self, replica, mean):
        import torch
        for g in replica.grads:
            t = torch.from_numpy(replica.bufs[g])
            self.dist.all_reduce(t)
            if mean:
                t /= self.n_ranks


def _one_step(handle, lr):
    handle.replica.set_values({"w": np.float32([0.5]), "learning_rate": np.float32([lr])})
    handle.set_batch(X, Y)
    handle.step()
    return handle.owner_loss_value(), float(handle.read_values("w")[0])


def test_single_shard_known_answer():
    rep = OracleReplica(W.linreg_update(4), W.linreg_sgd(), ["w"])
    h = par.DataParallel(rep, par.LocalExchange(), "sum")
    loss, w = _one_step(h, 0.05)
    assert abs(loss - 67.5) < 1e-4 and abs(w - 5.0) < 1e-5
    assert h.shard_seeds == [0]


def _gloo_rank(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rep = OracleReplica(W.linreg_update(4 // world), W.linreg_sgd(), ["w"])
        h = par.DataParallel(rep, GlooExchange(dist), "sum", base_seed=100)
        loss, w = _one_step(h, 0.05)
        # multi-step with mean reduction on a fresh batch (test/training/data_parallel.ml:61-83)
        h2 = par.DataParallel(rep, GlooExchange(dist), "mean")
        l1, _ = _one_step(h2, 0.02)
        h2.set_batch(np.float32([[5.], [6.], [7.], [8.]]), np.float32([[10.], [12.], [14.], [16.]]))
        h2.step()
        l2 = h2.owner_loss_value()
        q.put((rank, loss, w, h.shard_seeds, l1, l2, float(h2.read_values("w")[0])))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_single_shard():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, loss0, w0, seeds, l1, l2, wm0), (r1, loss1, w1, _, _, _, wm1) = out
    assert abs(loss0 - 11.25) < 1e-4            # the owner's half batch: x = 1, 2
    assert abs(w0 - 5.0) < 1e-5 and w0 == w1    # same parameters as the 1-shard step, on every replica
    assert seeds == [100, 101]
    assert np.isfinite(l1) and np.isfinite(l2) and wm0 == wm1


def _nccl_rank(rank, world, uid, q):
    """One rank of the two-GPU tests.  Whatever goes wrong is reported through the queue, and the
    communicator carries a timeout, so that a rank whose peer failed gives up instead of spinning
    inside a collective."""
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        from ocannl_b200 import backend as bk
        dev = bk.Device(rank)
        rep = par.DeviceReplica(dev, W.linreg_update(4 // world), W.linreg_sgd(), ["w"])
        ex = par.NcclExchange(dev, world, rank, uid)
        ex.set_timeout(60000)
        h = par.DataParallel(rep, ex, "sum")
        loss, w = _one_step(h, 0.05)
        h.sync_params_to_host()
        # the MLP update with the exchange carried by the routine, in buckets, beside the backward pass
        rows = 512
        mlp = par.DeviceReplica(dev, W.mlp_train_update(rows=rows // world), W.mlp_sgd(), W.MLP_PARAM_NAMES)
        buckets = ex.attach_overlap(mlp, mean=True)
        hm = par.DataParallel(mlp, ex, "mean", input_ident="x", target_ident="labels")
        x, onehot = W.mlp_inputs(rows=rows)
        mlp.set_values(dict(W.mlp_params(), learning_rate=np.float32([0.1])))
        hm.set_batch(x, onehot)
        for _ in range(3):               # the third run replays the captured graph
            hm.step()
        hm.sync_params_to_host()
        params = {k: W.load("bfloat16", hm.read_values(k)).astype(np.float32) for k in W.MLP_PARAM_NAMES}
        grads = {k: hm.read_values(k + "_grad") for k in W.MLP_PARAM_NAMES}
        q.put((rank, loss, w, len(buckets), params, grads))
        ex.free()
    except Exception as e:      # noqa: BLE001 - the parent must learn of any failure
        import traceback
        q.put((rank, "error", traceback.format_exc()))


def _run_ranks(target, args_of, n):
    """Starts n ranks, collects one message from each and never leaves a rank behind."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=args_of(r) + (q,)) for r in range(n)]
    for p in procs:
        p.start()
    try:
        out = sorted((q.get(timeout=300) for _ in procs), key=lambda m: m[0])
        for m in out:
            assert m[1] != "error", m[2]
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        return out
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
                if p.is_alive():
                    p.kill()


def _mlp_steps(device, exchange, overlap, graph=True, rows=256, steps=3):
    mlp = par.DeviceReplica(device, W.mlp_train_update(rows=rows), W.mlp_sgd(), W.MLP_PARAM_NAMES, graph=graph)
    if overlap:
        exchange.attach_overlap(mlp, mean=True)
    hm = par.DataParallel(mlp, exchange, "mean", input_ident="x", target_ident="labels")
    x, onehot = W.mlp_inputs(rows=rows)
    mlp.set_values(dict(W.mlp_params(), learning_rate=np.float32([0.1])))
    hm.set_batch(x, onehot)
    for _ in range(steps):
        hm.step()
    hm.sync_params_to_host()
    return {k: hm.read_values(k) for k in list(W.MLP_PARAM_NAMES) + [p + "_grad" for p in W.MLP_PARAM_NAMES]}


def _single_rank_overlap(q):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        from ocannl_b200 import backend as bk
        dev = bk.Device(0)
        plain = _mlp_steps(dev, par.LocalExchange(), False)
        out = {}
        for graph in (False, True):
            ex = par.NcclExchange(dev, 1, 0, par.NcclExchange.unique_id())
            ex.set_timeout(30000)
            got = _mlp_steps(dev, ex, True, graph=graph)
            # worst difference relative to the node's largest magnitude (bf16 parameters as bits -> values)
            worst = 0.0
            for k in plain:
                a = (W.load("bfloat16", plain[k]) if plain[k].dtype == np.uint16 else plain[k]).astype(np.float64)
                b = (W.load("bfloat16", got[k]) if got[k].dtype == np.uint16 else got[k]).astype(np.float64)
                worst = max(worst, float(np.abs(a - b).max() / max(np.abs(a).max(), 1e-30)))
            out[graph] = worst
            ex.free()
        q.put((0, out))
    except Exception:      # noqa: BLE001
        import traceback
        q.put((0, "error", traceback.format_exc()))


@pytest.mark.gpu
def test_overlapped_exchange_with_one_rank(device):
    """The exchange attached to the update routine (bucket allreduces on the communicator's stream,
    forked from and joined to the compute stream, also inside the captured graph), with a
    communicator of one rank: an average over one rank changes nothing, so parameters and gradients
    after three steps equal those of the run without an exchange, up to the last bits of the weight
    gradients that split-K adds in no fixed order."""
    out = _run_ranks(_single_rank_overlap, lambda r: (), 1)
    assert out[0][1][False] < 1e-3 and out[0][1][True] < 1e-3, out


@pytest.mark.gpu
def test_two_gpus_nccl_match_single_shard(device):
    from ocannl_b200 import backend as bk
    rep = par.DeviceReplica(device, W.linreg_update(4), W.linreg_sgd(), ["w"])
    h = par.DataParallel(rep, par.LocalExchange(), "sum")
    loss, w = _one_step(h, 0.05)
    assert abs(loss - 67.5) < 1e-4 and abs(w - 5.0) < 1e-5
    # the MLP on one shard: what two shards with an averaged exchange must reproduce
    rows = 512
    mlp = par.DeviceReplica(device, W.mlp_train_update(rows=rows), W.mlp_sgd(), W.MLP_PARAM_NAMES)
    hm = par.DataParallel(mlp, par.LocalExchange(), "mean", input_ident="x", target_ident="labels")
    x, onehot = W.mlp_inputs(rows=rows)
    mlp.set_values(dict(W.mlp_params(), learning_rate=np.float32([0.1])))
    hm.set_batch(x, onehot)
    for _ in range(3):
        hm.step()
    hm.sync_params_to_host()
    one = {k: W.load("bfloat16", hm.read_values(k)).astype(np.float32) for k in W.MLP_PARAM_NAMES}
    one_g = {k: hm.read_values(k + "_grad") for k in W.MLP_PARAM_NAMES}
    assert mlp.gradient_buckets(3) and len(mlp.gradient_buckets(3)) == 2      # (w2, b2, w_out) then (w1, b1)
    if bk.num_devices() < 2:
        pytest.skip("needs two GPUs")
    uid = par.NcclExchange.unique_id()
    out = _run_ranks(_nccl_rank, lambda r: (r, 2, uid), 2)
    assert abs(out[0][1] - 11.25) < 1e-4
    assert abs(out[0][2] - 5.0) < 1e-5 and out[0][2] == out[1][2]
    assert out[0][3] == 2
    for k in W.MLP_PARAM_NAMES:
        # both replicas hold the same parameters, bit for bit, and the same reduced gradients
        assert np.array_equal(out[0][4][k], out[1][4][k]), k
        assert np.array_equal(out[0][5][k], out[1][5][k]), k
        # and they are those of the one-shard run up to the rounding of bf16 activations: a mean
        # over two half batches adds in another order
        g1, g2 = one_g[k].astype(np.float64), out[0][5][k].astype(np.float64)
        assert np.linalg.norm(g1 - g2) <= 5e-2 * np.linalg.norm(g1), k
        assert np.abs(one[k] - out[0][4][k]).max() <= 2.0 ** -7 * np.abs(one[k]).max() + 1e-6, k


@pytest.mark.gpu
def test_all_shards_in_one_process(device):
    """The reference's arrangement: one process holds every shard (lib/parallel.ml:166-208).  The
    known answers of test/training/data_parallel.expected with one and -- where two GPUs are
    visible -- two shards: owner losses 67.5 / 11.25, w = 5.0 on every replica."""
    from ocannl_b200 import backend as bk

    def run(devs):
        h = par.data_parallel(devs, lambda rows: W.linreg_update(rows), W.linreg_sgd(), ["w"], 4, "sum", base_seed=7)
        for r in h.replicas:
            r.set_values({"w": np.float32([0.5]), "learning_rate": np.float32([0.05])})
        h.set_batch(X, Y)
        h.step()
        h.sync_params_to_host()
        out = h.owner_loss_value(), [float(h.read_values("w", i)[0]) for i in range(h.n_shards)], h.shard_seeds
        h.free()
        return out

    loss, ws, seeds = run([device])
    assert abs(loss - 67.5) < 1e-4 and abs(ws[0] - 5.0) < 1e-5 and seeds == [7]
    with pytest.raises(ValueError):
        par.data_parallel([device, device, device], lambda rows: W.linreg_update(rows), W.linreg_sgd(), ["w"], 4)
    if bk.num_devices() < 2:
        pytest.skip("needs two GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    loss, ws, seeds = run([device, bk.Device(1)])
    assert abs(loss - 11.25) < 1e-4 and all(abs(w - 5.0) < 1e-5 for w in ws) and ws[0] == ws[1] and seeds == [7, 8]
