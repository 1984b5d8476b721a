"""Data-parallel driver: batch sharding and the gradient exchange.

Mirrors `Parallel` of the reference (lib/parallel.ml): `shard_along` / `gather` (:51-110) and the
`data_parallel` handle (:112-141: `step`, `grad_sync`, `set_batch`, `owner_loss_value`,
`read_values`, `owner_params`, `shard_seeds`).  The reference keeps all shards in one process and
moves every parameter gradient to an "owner" shard through merge-buffer copies, updates there and
broadcasts the parameters back (:247-304).  Here every shard is one process on one GPU; the
exchange is ONE allreduce (sum, or average for `reduction="mean"`) over the contiguous range that
holds all parameter gradients, after which every shard applies the same SGD step to its own
replica — parameters stay identical without a broadcast.  The owner is shard 0, whose loss is the
one `owner_loss_value` reports, as in the reference (:364-366).

The driver is written against two small interfaces so that the same code runs with GPU replicas
over NCCL (`DeviceReplica` + `NcclExchange`) and, in the CPU tests, with stand-in replicas over
gloo ranks.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from . import backend as bk
from .low_level import Routine as IrRoutine, Tnode


# ------------------------------------------------------------------ shard_along / gather
def shard_along(values: np.ndarray, n_shards: int, axis: int = 0) -> List[np.ndarray]:
    """Contiguous row blocks of the leading axis, copied (lib/parallel.ml:51-79)."""
    if n_shards <= 0:
        raise ValueError("Parallel.shard_along: n_shards must be > 0")
    if axis != 0:
        raise ValueError("Parallel.shard_along: only axis=0 (leftmost batch axis) supported, got %d" % axis)
    values = np.asarray(values)
    if values.ndim == 0:
        raise ValueError("Parallel.shard_along: scalar tensor has no batch axis to shard")
    batch = values.shape[0]
    if batch % n_shards != 0:
        raise ValueError("Parallel.shard_along: batch size %d not divisible by n_shards %d" % (batch, n_shards))
    sub = batch // n_shards
    return [np.ascontiguousarray(values[k * sub:(k + 1) * sub]) for k in range(n_shards)]


def gather(shards: Sequence[np.ndarray], axis: int = 0) -> np.ndarray:
    """Inverse of `shard_along` (lib/parallel.ml:84-110)."""
    if len(shards) == 0:
        raise ValueError("Parallel.gather: empty shards array")
    if axis != 0:
        raise ValueError("Parallel.gather: only axis=0 (leftmost batch axis) supported, got %d" % axis)
    rest = shards[0].shape[1:]
    for i, s in enumerate(shards):
        if s.ndim == 0 or s.shape[1:] != rest:
            raise ValueError("Parallel.gather: shard %d has incompatible shape for axis-0 gather" % i)
    return np.concatenate(list(shards), axis=0)


# ------------------------------------------------------------------ exchange
class NcclExchange:
    """Gradient allreduce over NVLink through the library's NCCL binding (`b200_allreduce`);
    one communicator rank per process and device."""

    def __init__(self, device: bk.Device, n_ranks: int, rank: int, unique_id: bytes):
        self.device, self.n_ranks, self.rank = device, n_ranks, rank
        h = ctypes.c_void_p()
        bk.check(bk.lib().b200_comm_init_rank(device.h, ctypes.c_int(n_ranks), ctypes.c_int(rank),
                                              ctypes.c_char_p(unique_id), ctypes.byref(h)))
        self.h = h

    @staticmethod
    def unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        bk.check(bk.lib().b200_comm_unique_id(buf))
        return buf.raw

    def allreduce(self, replica: "DeviceReplica", mean: bool):
        if self.overlapped:
            return       # the update routine carries the exchange (attach_overlap)
        pool, offset, count = replica.grad_range
        bk.check(bk.lib().b200_allreduce(self.h, ctypes.c_int(pool), ctypes.c_size_t(offset), ctypes.c_size_t(count),
                                         ctypes.c_int(0), ctypes.c_int(1 if mean else 0)))

    overlapped = False

    def attach_overlap(self, replica: "DeviceReplica", mean: bool, max_buckets: int = 3):
        """Makes the exchange part of the update routine: the gradient range is cut into at most
        `max_buckets` buckets of similar size in the order back-propagation completes them (last
        layers first); each bucket's allreduce starts on the communicator's stream as soon as the
        last kernel writing into it is queued and runs beside the rest of the backward pass
        (b200_routine_overlap_allreduce).  `grad_sync` then has nothing left to do."""
        buckets = replica.gradient_buckets(max_buckets)
        n = len(buckets)
        pools = (ctypes.c_int * n)(*[b[0] for b in buckets])
        offs = (ctypes.c_size_t * n)(*[b[1] for b in buckets])
        counts = (ctypes.c_size_t * n)(*[b[2] for b in buckets])
        bk.check(bk.lib().b200_routine_overlap_allreduce(replica.update.h, self.h, ctypes.c_int(n), pools, offs, counts,
                                                         ctypes.c_int(0), ctypes.c_int(1 if mean else 0)))
        if replica.graph:
            replica.update.use_graph(True)
        self.overlapped = True
        return buckets

    def set_timeout(self, milliseconds: int):
        """`await` polls for asynchronous NCCL errors and aborts the communicator when one shows up
        or the stream stays busy this long (a rank that left)."""
        bk.check(bk.lib().b200_comm_set_timeout(self.h, ctypes.c_longlong(milliseconds)))

    def free(self):
        if self.h:
            bk.lib().b200_comm_free(self.h)
            self.h = None


class LocalExchange:
    """Single shard: nothing to exchange."""
    n_ranks, rank = 1, 0

    def allreduce(self, replica, mean: bool):
        return None


# ------------------------------------------------------------------ replicas
class DeviceReplica:
    """One shard on one GPU: the forward+backward routine (`Train.grad_update`, lib/train.ml:61-73)
    and the optimizer routine (`Train.sgd_update`, :76-90) linked into one context.  All parameter
    gradients are allocated first, back to back in one pool, so that the exchange is a single
    allreduce over [first gradient, last gradient]."""

    def __init__(self, device: bk.Device, update: IrRoutine, sgd: IrRoutine, params: Sequence[str],
                 grad_suffix: str = "_grad", loss: str = "loss", graph: bool = True):
        self.device = device
        self.params = list(params)
        self.loss_ident = loss
        grads = [t for p in self.params for t in update.tnodes if t.ident == p + grad_suffix]
        if len(grads) != len(self.params):
            raise bk.UserError(-5, "data_parallel: every parameter needs a gradient node '<param>%s'" % grad_suffix)
        for g in grads:
            if g.prec != "single":
                raise bk.UserError(-5, "data_parallel: gradient '%s' must be single precision" % g.ident)
        ctx = bk.Context(device).allocate(grads)
        pool = ctx.arrays[grads[0].ident][0]
        first = min(ctx.arrays[g.ident][1] for g in grads)
        last = max(ctx.arrays[g.ident][1] + g.size_in_bytes for g in grads)
        self.grad_range = (pool, first, (last - first) // 4)
        # gradients in memory order with their byte ranges (parameters are declared first layer first)
        self.grad_layout = sorted(((ctx.arrays[g.ident][1], g.size_in_bytes, g.ident) for g in grads))
        self.graph = graph
        self.update_code, self.sgd_code = bk.Code(update), bk.Code(sgd)
        self.update = ctx.link(self.update_code)
        self.sgd = self.update.context.link(self.sgd_code)
        self.context = self.sgd.context
        if graph:
            self.update.use_graph(True)
            self.sgd.use_graph(True)

    def gradient_buckets(self, max_buckets: int = 3):
        """Contiguous (pool, byte offset, element count) ranges covering all gradients, at most
        `max_buckets` of them, listed in the order back-propagation completes them: the gradients
        of the last layers lie last in memory and are finished first.  Cuts are made where the
        bytes gathered from the end pass the next multiple of total / max_buckets."""
        pool = self.grad_range[0]
        total = sum(size for _, size, _ in self.grad_layout)
        out, hi, acc, k = [], None, 0, 1
        for off, size, _ in reversed(self.grad_layout):
            if hi is None:
                hi = off + size
            acc += size
            if acc >= k * total / max_buckets or off == self.grad_layout[0][0]:
                out.append((pool, off, (hi - off) // 4))
                hi = None
                while acc >= k * total / max_buckets:
                    k += 1
        return out

    def set_values(self, values: Dict[str, np.ndarray]):
        for k, v in values.items():
            self.context.from_host(k, v)

    def forward_backward(self, **static):
        self.update.run(**static)

    def optimizer_step(self, **static):
        self.sgd.run(**static)

    def read(self, ident: str) -> np.ndarray:
        return self.context.to_host(ident)

    def await_(self):
        self.device.await_()


class DataParallel:
    """The handle of `Parallel.data_parallel` (lib/parallel.ml:112-141) for this process's shard."""

    def __init__(self, replica, exchange, reduction: str = "sum", base_seed: int = 0,
                 input_ident: str = "x", target_ident: str = "y"):
        if reduction not in ("sum", "mean"):
            raise ValueError("Parallel.data_parallel: reduction must be 'sum' or 'mean'")
        self.replica, self.exchange = replica, exchange
        self.n_shards = exchange.n_ranks
        self.rank = exchange.rank
        self.mean = reduction == "mean"
        self.shard_seeds = [base_seed + i for i in range(self.n_shards)]
        self.seed = self.shard_seeds[self.rank]
        self.input_ident, self.target_ident = input_ident, target_ident
        self.owner_params = list(replica.params)

    def set_batch(self, inputs: np.ndarray, targets: np.ndarray):
        """Scatter a logical batch: this shard keeps its contiguous block of rows."""
        xs = shard_along(inputs, self.n_shards)
        ys = shard_along(targets, self.n_shards)
        self.replica.set_values({self.input_ident: xs[self.rank], self.target_ident: ys[self.rank]})

    def grad_sync(self):
        self.exchange.allreduce(self.replica, self.mean)

    def step(self, **static):
        self.replica.forward_backward(**static)
        self.grad_sync()
        self.replica.optimizer_step(**static)

    def owner_loss_value(self) -> float:
        """The loss of this process's shard; on rank 0 that is the owner's loss."""
        return float(self.replica.read(self.replica.loss_ident).reshape(-1)[0])

    def sync_params_to_host(self):
        self.replica.await_()

    def read_values(self, ident: str) -> np.ndarray:
        return self.replica.read(ident)


# ------------------------------------------------------------------ all shards in one process
class Handle:
    """`Parallel.handle` (lib/parallel.ml:112-141) with every shard held by this process, the
    reference's own arrangement: `n_shards`, `step`, `grad_sync`, `set_batch`, `owner_loss_value`,
    `sync_params_to_host`, `read_values`, `owner_params`, `shard_seeds`.  The owner is shard 0.
    The reference moves each gradient to the owner through merge-buffer copies, updates there
    and broadcasts the parameters (:247-304); here `grad_sync` is one grouped NCCL allreduce over
    the shards' contiguous gradient ranges and every shard applies the optimizer routine itself."""

    def __init__(self, replicas: Sequence[DeviceReplica], reduction: str, base_seed: int, input_ident: str, target_ident: str):
        if reduction not in ("sum", "mean"):
            raise ValueError("Parallel.data_parallel: reduction must be 'sum' or 'mean'")
        self.replicas = list(replicas)
        self.n_shards = len(self.replicas)
        self.mean = reduction == "mean"
        self.shard_seeds = [base_seed + i for i in range(self.n_shards)]
        self.input_ident, self.target_ident = input_ident, target_ident
        self.owner_params = list(self.replicas[0].params)
        self.comms = None
        if self.n_shards > 1:
            n = self.n_shards
            devs = (ctypes.c_void_p * n)(*[r.device.h for r in self.replicas])
            out = (ctypes.c_void_p * n)()
            bk.check(bk.lib().b200_comm_init_all(ctypes.c_int(n), devs, out))
            self.comms = out

    def set_batch(self, inputs: np.ndarray, targets: np.ndarray):
        xs, ys = shard_along(inputs, self.n_shards), shard_along(targets, self.n_shards)
        for r, x, y in zip(self.replicas, xs, ys):
            r.set_values({self.input_ident: x, self.target_ident: y})

    def grad_sync(self):
        if self.comms is None:
            return
        n = self.n_shards
        count = self.replicas[0].grad_range[2]
        pools = (ctypes.c_int * n)(*[r.grad_range[0] for r in self.replicas])
        offs = (ctypes.c_size_t * n)(*[r.grad_range[1] for r in self.replicas])
        bk.check(bk.lib().b200_allreduce_all(ctypes.c_int(n), self.comms, pools, offs, ctypes.c_size_t(count), ctypes.c_int(0),
                                             ctypes.c_int(1 if self.mean else 0)))

    def step(self, **static):
        for r in self.replicas:          # launch every shard before waiting for any
            r.forward_backward(**static)
        self.grad_sync()
        for r in self.replicas:
            r.optimizer_step(**static)

    def owner_loss_value(self) -> float:
        return float(self.replicas[0].read(self.replicas[0].loss_ident).reshape(-1)[0])

    def sync_params_to_host(self):
        for r in self.replicas:
            r.await_()

    def read_values(self, ident: str, shard: int = 0) -> np.ndarray:
        return self.replicas[shard].read(ident)

    def free(self):
        if self.comms is not None:
            for c in self.comms:
                bk.lib().b200_comm_free(ctypes.c_void_p(c))
            self.comms = None


def data_parallel(devices: Sequence[bk.Device], update_of_rows: Callable[[int], IrRoutine], sgd: IrRoutine, params: Sequence[str],
                  batch_rows: int, reduction: str = "sum", base_seed: int = 0, input_ident: str = "x",
                  target_ident: str = "y", loss: str = "loss") -> Handle:
    """`Parallel.data_parallel` (lib/parallel.ml:166-383): one replica per device in this process,
    each over `batch_rows / n` rows (the batch must divide evenly, :51-66), seeds `base_seed + i`.
    `update_of_rows(rows)` builds the forward+backward routine of a shard of that many rows."""
    n = len(devices)
    if n <= 0:
        raise ValueError("Parallel.data_parallel: needs at least one device")
    if batch_rows % n != 0:
        raise ValueError("Parallel.shard_along: batch size %d not divisible by n_shards %d" % (batch_rows, n))
    reps = [DeviceReplica(d, update_of_rows(batch_rows // n), sgd, params, loss=loss) for d in devices]
    return Handle(reps, reduction, base_seed, input_ident, target_ident)
