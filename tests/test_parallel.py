"""Data-parallel driver: sharding helpers, the reference's known answers for a 1-shard and a
2-shard step (test/training/data_parallel.expected: losses 67.5 / 11.25, w = 5.0 both ways),
over gloo ranks on CPU (replicas run the CPU oracle) and over NCCL on two GPUs."""
import os
import sys

import numpy as np
import pytest

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
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from ocannl_b200 import backend as bk
    dev = bk.Device(rank)
    rep = par.DeviceReplica(dev, W.linreg_update(4 // world), W.linreg_sgd(), ["w"])
    ex = par.NcclExchange(dev, world, rank, uid)
    h = par.DataParallel(rep, ex, "sum")
    loss, w = _one_step(h, 0.05)
    h.sync_params_to_host()
    q.put((rank, loss, w))
    ex.free()


@pytest.mark.gpu
def test_two_gpus_nccl_match_single_shard(device):
    from ocannl_b200 import backend as bk
    rep = par.DeviceReplica(device, W.linreg_update(4), W.linreg_sgd(), ["w"])
    h = par.DataParallel(rep, par.LocalExchange(), "sum")
    loss, w = _one_step(h, 0.05)
    assert abs(loss - 67.5) < 1e-4 and abs(w - 5.0) < 1e-5
    if bk.num_devices() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    uid = par.NcclExchange.unique_id()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_rank, args=(r, 2, uid, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert abs(out[0][1] - 11.25) < 1e-4
    assert abs(out[0][2] - 5.0) < 1e-5 and out[0][2] == out[1][2]
