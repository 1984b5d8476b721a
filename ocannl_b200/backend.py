"""ctypes binding of libb200.so and a host-side mirror of arrayjit's backend interface.

The classes follow the user-facing signatures of arrayjit/lib/backend_intf.ml:
`Backend.compile` / `link` (:319-336), `routine` (:59-70), `context` (:134-149), device
`await` / `all_work` (:97-126) and the host copies `from_host` / `to_host`
(arrayjit/lib/backends.ml:113-158).  `Context.link` restates `Raise_backend.allocate_delta`
(arrayjit/lib/backends.ml:529-614): nodes of the routine that the parent context does not
hold yet are bump-packed into one new pool, zero-initialised unless the routine zeroes them
itself, and the child context records their {pool, offset}.

Everything that computes goes through the C ABI of include/b200.h; when the library or a
GPU is missing the calls raise — there is no CPU fallback.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .low_level import PREC_BYTES, Routine as IrRoutine, Tnode

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200.so")

NP_DTYPE = {"byte": np.uint8, "uint16": np.uint16, "int32": np.int32, "uint32": np.uint32,
            "int64": np.int64, "uint64": np.uint64, "half": np.float16, "bfloat16": np.uint16,
            "fp8": np.uint8, "single": np.float32, "double": np.float64,
            # four 32-bit words per element: arrays of this precision get a trailing axis of 4
            "uint4x32": np.dtype((np.uint32, (4,)))}


class B200Error(RuntimeError):
    """Non-zero status from the C ABI; `.code` < 0 is a B200_E_* value, > 0 a CUDA /
    NVRTC / NCCL result."""

    def __init__(self, code: int, msg: str):
        super().__init__("b200 error %d: %s" % (code, msg))
        self.code = code


class UserError(B200Error):
    """Utils.User_error of the reference: bad static index, missing binding."""


class Binding(ctypes.Structure):
    _fields_ = [("tn_id", ctypes.c_int32), ("pool_id", ctypes.c_int32), ("offset", ctypes.c_uint64)]


_lib = None


def lib() -> ctypes.CDLL:
    """Loads libb200.so (built in-tree by `python -m ocannl_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(-2, "libb200.so is not built: run `python -m ocannl_b200.build`")
        L = ctypes.CDLL(LIB_PATH)
        L.b200_last_error.restype = ctypes.c_char_p
        L.b200_version.restype = ctypes.c_char_p
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = lib().b200_last_error().decode(errors="replace")
        raise (UserError if rc == -5 else B200Error)(rc, msg)


def _vp(x) -> ctypes.c_void_p:
    return ctypes.c_void_p(x)


class Event:
    def __init__(self, h):
        self.h = h

    def sync(self):
        check(lib().b200_event_sync(self.h))

    def is_done(self) -> bool:
        d = ctypes.c_int(0)
        check(lib().b200_event_query(self.h, ctypes.byref(d)))
        return bool(d.value)

    def elapsed_ms(self, later: "Event") -> float:
        ms = ctypes.c_float(0)
        check(lib().b200_event_elapsed_ms(self.h, later.h, ctypes.byref(ms)))
        return ms.value

    def free(self):
        if self.h:
            lib().b200_event_free(self.h)
            self.h = None


class Device:
    """One GPU with its stream and pool table (Backend_intf.device)."""

    def __init__(self, ordinal: int = 0):
        h = ctypes.c_void_p()
        check(lib().b200_device_open(ctypes.c_int(ordinal), ctypes.byref(h)))
        self.h = h
        self.ordinal = ordinal
        self._next_pool = 1            # pool id 0 is the merge buffer (backend_intf.ml:131-132)

    def props(self) -> dict:
        buf = ctypes.create_string_buffer(1024)
        check(lib().b200_device_props(self.h, buf, ctypes.c_size_t(1024)))
        return json.loads(buf.value.decode())

    def alloc_pool(self, size_in_bytes: int, pool_id: Optional[int] = None, alignment: int = 256) -> int:
        if pool_id is None:
            pool_id = self._next_pool
            self._next_pool += 1
        check(lib().b200_pool_alloc(self.h, ctypes.c_int(pool_id), ctypes.c_size_t(size_in_bytes),
                                    ctypes.c_size_t(alignment)))
        return pool_id

    def free_pool(self, pool_id: int):
        check(lib().b200_pool_free(self.h, ctypes.c_int(pool_id)))

    def memset_zero(self, pool_id: int, offset: int, size_in_bytes: int):
        check(lib().b200_pool_memset0(self.h, ctypes.c_int(pool_id), ctypes.c_size_t(offset),
                                      ctypes.c_size_t(size_in_bytes)))

    def pool_address(self, pool_id: int) -> Tuple[int, int]:
        p, n = ctypes.c_uint64(0), ctypes.c_size_t(0)
        check(lib().b200_pool_address(self.h, ctypes.c_int(pool_id), ctypes.byref(p), ctypes.byref(n)))
        return p.value, n.value

    def from_host(self, pool_id: int, offset: int, arr: np.ndarray):
        assert arr.flags["C_CONTIGUOUS"]
        check(lib().b200_h2d(self.h, ctypes.c_int(pool_id), ctypes.c_size_t(offset), _vp(arr.ctypes.data),
                             ctypes.c_size_t(arr.nbytes)))

    def to_host(self, pool_id: int, offset: int, arr: np.ndarray):
        assert arr.flags["C_CONTIGUOUS"] and arr.flags["WRITEABLE"]
        check(lib().b200_d2h(self.h, ctypes.c_int(pool_id), ctypes.c_size_t(offset), _vp(arr.ctypes.data),
                             ctypes.c_size_t(arr.nbytes)))

    def device_to_device(self, dst_pool: int, dst_offset: int, src: "Device", src_pool: int, src_offset: int, nbytes: int):
        """Copy between pools of one device or of two (`device_to_device ~into_merge_buffer:No`,
        arrayjit/lib/cuda_backend.ml:289-314), ordered after the work queued on the source."""
        check(lib().b200_d2d(self.h, ctypes.c_int(dst_pool), ctypes.c_size_t(dst_offset), src.h, ctypes.c_int(src_pool),
                             ctypes.c_size_t(src_offset), ctypes.c_size_t(nbytes)))

    def merge_copy(self, src: "Device", src_pool: int, src_offset: int, nbytes: int):
        """`device_to_device ~into_merge_buffer:Copy`: the source node lands in this device's merge
        buffer (pool 0, grown as needed), where a routine's `Get_merge_buffer` reads it."""
        check(lib().b200_merge_copy(self.h, src.h, ctypes.c_int(src_pool), ctypes.c_size_t(src_offset), ctypes.c_size_t(nbytes)))

    def all_work(self) -> Event:
        e = ctypes.c_void_p()
        check(lib().b200_event_record(self.h, ctypes.byref(e)))
        return Event(e)

    def will_wait_for(self, ev: Event):
        check(lib().b200_stream_wait(self.h, ev.h))

    def await_(self):
        check(lib().b200_await(self.h))

    def is_idle(self) -> bool:
        d = ctypes.c_int(0)
        check(lib().b200_is_idle(self.h, ctypes.byref(d)))
        return bool(d.value)

    def set_async_uploads(self, on: bool = True):
        """from_host copies on a second stream (see b200_set_async_uploads in include/b200.h)."""
        check(lib().b200_set_async_uploads(self.h, ctypes.c_int(1 if on else 0)))

    def stream_handle(self) -> int:
        s = ctypes.c_uint64(0)
        check(lib().b200_stream_handle(self.h, ctypes.byref(s)))
        return s.value

    def sum_f32_static(self, in_pool: int, in_offset: int, count: int, out_pool: int, out_offset: int):
        """Sum of `count` floats, written as one float, without any allocation at call time
        (scratch is a fixed 4 KiB array inside the library's device image; count <= 2**26).
        For callers that must not touch the device allocator while running; calls that overlap
        on the GPU share that array and race, stream-ordered calls are safe."""
        check(lib().b200_sum_f32_static(self.h, ctypes.c_int(in_pool), ctypes.c_size_t(in_offset),
                                        ctypes.c_size_t(count), ctypes.c_int(out_pool), ctypes.c_size_t(out_offset)))

    def get_used_memory(self) -> int:
        n = ctypes.c_size_t(0)
        check(lib().b200_used_memory(self.h, ctypes.byref(n)))
        return n.value

    def get_debug_info(self) -> dict:
        buf = ctypes.create_string_buffer(1024)
        check(lib().b200_debug_info(self.h, buf, ctypes.c_size_t(1024)))
        return json.loads(buf.value.decode())


def num_devices() -> int:
    n = ctypes.c_int(0)
    check(lib().b200_num_devices(ctypes.byref(n)))
    return n.value


class PinnedBuffer:
    """Page-locked host memory viewed as a numpy array (for from_host / to_host)."""

    def __init__(self, shape, dtype):
        self.nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = ctypes.c_void_p()
        check(lib().b200_host_alloc(ctypes.c_size_t(max(self.nbytes, 1)), ctypes.byref(p)))
        self.ptr = p
        raw = (ctypes.c_char * max(self.nbytes, 1)).from_address(p.value)
        self.array = np.frombuffer(raw, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def free(self):
        if self.ptr:
            self.array = None
            lib().b200_host_free(self.ptr)
            self.ptr = None


class Code:
    """Device-independent compiled routine (`Backend.compile`)."""

    def __init__(self, ir: IrRoutine, options: Optional[str] = None, name: Optional[str] = None):
        self.ir = ir
        text = ir.to_b200ir().encode()
        h = ctypes.c_void_p()
        check(lib().b200_compile((name or "").encode(), text, ctypes.c_size_t(len(text)),
                                 options.encode() if options else None, ctypes.byref(h)))
        self.h = h

    def info(self) -> dict:
        buf = ctypes.create_string_buffer(1 << 16)
        check(lib().b200_code_info(self.h, buf, ctypes.c_size_t(1 << 16)))
        return json.loads(buf.value.decode())

    def source(self, stage: int = -1) -> str:
        need = ctypes.c_size_t(0)
        check(lib().b200_code_source(self.h, ctypes.c_int(stage), None, ctypes.c_size_t(0), ctypes.byref(need)))
        buf = ctypes.create_string_buffer(need.value)
        check(lib().b200_code_source(self.h, ctypes.c_int(stage), buf, ctypes.c_size_t(need.value), None))
        return buf.value.decode()

    def free(self):
        if self.h:
            lib().b200_code_free(self.h)
            self.h = None


def compile(ir: IrRoutine, options: Optional[str] = None) -> Code:  # noqa: A001 (mirrors Backend.compile)
    return Code(ir, options)


POOL_CAP = 0x1_0000_0000   # bytes per pool while offsets are 32-bit (arrayjit/lib/backends.ml:536)


def plan_pool_segments(items: Sequence[Tuple[int, int]], cap: int = POOL_CAP, what: str = "allocate_delta",
                       names: Optional[Sequence[str]] = None) -> Tuple[List[Tuple[int, int]], List[int]]:
    """`Backend_utils.plan_pool_segments` (arrayjit/lib/backends.ml:22-51): lays `(size, alignment)`
    items out in order; an item that would carry a pool past `cap` bytes opens a new pool at
    offset 0.  Returns `[(segment, offset)]` per item and the byte size of every segment; an item
    larger than the cap is a user error."""
    seg, bump, closed, out = 0, 0, [], []
    for i, (size, align) in enumerate(items):
        if size > cap:
            raise UserError(-5, "%s: tensor node %s needs %d bytes, over the %d-byte per-pool cap; set large_models" % (
                what, names[i] if names else i, size, cap))
        off = bump if align <= 1 else (bump + align - 1) // align * align
        if off + size > cap:
            closed.append(bump)
            seg += 1
            bump = size
            out.append((seg, 0))
        else:
            bump = off + size
            out.append((seg, off))
    return out, (closed + [bump]) if items else []


class Context:
    """`Backend_intf.context`: a device plus the {node -> (pool, offset)} map of the nodes it
    holds.  Contexts are persistent: `link` returns a routine whose `.context` is the child.

    `packing` chooses how `link` lays out the nodes the parent does not hold yet:
      "reference"  as `Raise_backend.allocate_delta` does (arrayjit/lib/backends.ml:529-614): working
                   nodes and read-only nodes go to separate pools, every node aligned to its ELEMENT
                   size only, pools cut at 4 GiB unless `large_models`, read-only nodes shared per
                   device by identifier;
      "aligned"    one pool, every node at a multiple of 256 bytes (the default of this mirror:
                   every stage then keeps its fastest form)."""

    def __init__(self, device: Device, arrays: Optional[Dict[str, Tuple[int, int, Tnode]]] = None,
                 packing: str = "aligned", large_models: bool = False):
        self.device = device
        self.arrays: Dict[str, Tuple[int, int, Tnode]] = dict(arrays or {})   # ident -> (pool, offset, tn)
        self.packing = packing
        self.large_models = large_models

    def _child(self, arrays) -> "Context":
        return Context(self.device, arrays, self.packing, self.large_models)

    def allocate(self, tnodes: Sequence[Tnode]) -> "Context":
        """Child context that also holds `tnodes`, packed back to back in one new zeroed pool
        (how the data-parallel driver keeps all gradients in one contiguous range)."""
        new = [t for t in tnodes if t.ident not in self.arrays]
        arrays = dict(self.arrays)
        if new:
            offs, total = [], 0
            for t in new:
                total = (total + 255) // 256 * 256
                offs.append(total)
                total += t.size_in_bytes
            pool = self.device.alloc_pool(max(total, 1))
            self.device.memset_zero(pool, 0, max(total, 1))
            for t, o in zip(new, offs):
                arrays[t.ident] = (pool, o, t)
        return self._child(arrays)

    def _pack_reference(self, group: List[Tnode], arrays, zero: bool = True):
        if not group:
            return
        cap = (1 << 62) if self.large_models else POOL_CAP
        items = [(t.size_in_bytes, PREC_BYTES[t.prec]) for t in group]
        where, sizes = plan_pool_segments(items, cap, "allocate_delta", [t.ident for t in group])
        pools = []
        for seg, size in enumerate(sizes):
            align = max(PREC_BYTES[t.prec] for t, (s, _) in zip(group, where) if s == seg)
            pools.append(self.device.alloc_pool(max(size, 1), alignment=align))
        for t, (seg, off) in zip(group, where):
            if zero and not t.zero_init:
                self.device.memset_zero(pools[seg], off, t.size_in_bytes)
            arrays[t.ident] = (pools[seg], off, t)

    def link(self, code: Code) -> "Routine":
        dev = self.device
        new: List[Tnode] = [t for t in code.ir.params() if t.ident not in self.arrays]
        arrays = dict(self.arrays)
        if new and self.packing == "reference":
            cache = dev.__dict__.setdefault("constant_buffer_cache", {})
            working = [t for t in new if not t.read_only]
            constants = [t for t in new if t.read_only]
            self._pack_reference(working, arrays)
            fresh = []
            for t in constants:
                hit = cache.get(t.ident)
                if hit is not None and hit[2].prec == t.prec and tuple(hit[2].dims) == tuple(t.dims):
                    arrays[t.ident] = hit
                else:
                    fresh.append(t)
            self._pack_reference(fresh, arrays)
            for t in fresh:
                cache[t.ident] = arrays[t.ident]
        elif new:
            # bump-pack the delta into one pool at 256-byte multiples
            offs, total = [], 0
            for t in new:
                align = 256
                total = (total + align - 1) // align * align
                offs.append(total)
                total += t.size_in_bytes
            pool = dev.alloc_pool(max(total, 1))
            dev.memset_zero(pool, 0, max(total, 1))
            for t, o in zip(new, offs):
                arrays[t.ident] = (pool, o, t)
        for t in code.ir.params():
            have = arrays[t.ident][2]
            if have.prec != t.prec or tuple(have.dims) != tuple(t.dims):
                raise UserError(-5, "link: node '%s' is held with another precision or shape" % t.ident)
        params = code.ir.params()
        binds = (Binding * max(len(params), 1))()
        for i, t in enumerate(params):
            pool, off, _ = arrays[t.ident]
            binds[i] = Binding(t.id, pool, off)
        h = ctypes.c_void_p()
        check(lib().b200_link(dev.h, code.h, binds, ctypes.c_int(len(params)), ctypes.byref(h)))
        return Routine(self._child(arrays), code, h)

    # ---- host access (Context.set_values / get_values, arrayjit/lib/context.ml:322-395)
    def from_host(self, ident: str, arr: np.ndarray):
        pool, off, t = self.arrays[ident]
        words = 4 if t.prec == "uint4x32" else 1
        a = np.ascontiguousarray(arr, dtype=np.uint32 if words == 4 else NP_DTYPE[t.prec]).reshape(-1)
        if a.size != t.num_elems * words:
            raise UserError(-5, "from_host: '%s' has %d elements, got %d" % (ident, t.num_elems, a.size))
        self.device.from_host(pool, off, a)
        self.device.await_()     # the staging array may be a temporary

    def to_host(self, ident: str) -> np.ndarray:
        pool, off, t = self.arrays[ident]
        out = np.empty(t.dims if t.dims else (1,), NP_DTYPE[t.prec])
        self.device.to_host(pool, off, out)
        self.device.await_()
        return out


class Routine:
    """`Backend_intf.routine`: a linked routine; `run` schedules it on the device stream
    (`Task.run routine.schedule`, lib/train.ml:42)."""

    def __init__(self, context: Context, code: Code, h):
        self.context = context
        self.code = code
        self.h = h
        self.static_syms = [s for s, _ in code.ir.static]

    def run(self, **static):
        n = len(self.static_syms)
        vals = (ctypes.c_int64 * max(n, 1))(*[int(static[s]) for s in self.static_syms])
        check(lib().b200_launch(self.h, vals, ctypes.c_int(n)))

    def info(self) -> dict:
        """The plan that runs: the code's, or a re-planned variant of it when the bound addresses
        ruled out a stage's aligned form (b200_routine_info)."""
        buf = ctypes.create_string_buffer(1 << 16)
        check(lib().b200_routine_info(self.h, buf, ctypes.c_size_t(1 << 16)))
        return json.loads(buf.value.decode())

    def use_graph(self, on: bool = True):
        check(lib().b200_routine_use_graph(self.h, ctypes.c_int(int(on))))

    def kernels_per_run(self) -> int:
        k = ctypes.c_int64(0)
        check(lib().b200_routine_launch_count(self.h, ctypes.byref(k)))
        return k.value

    def profile(self, on: bool = True):
        check(lib().b200_routine_profile(self.h, ctypes.c_int(int(on))))

    def stage_times(self):
        """[(total_ms, runs)] per stage, over the runs made while profiling was on."""
        out = []
        for i in range(len(self.info()["stages"])):
            ms, n = ctypes.c_float(0), ctypes.c_int(0)
            check(lib().b200_routine_stage_time(self.h, ctypes.c_int(i), ctypes.byref(ms), ctypes.byref(n)))
            out.append((ms.value, n.value))
        return out

    def free(self):
        if self.h:
            lib().b200_routine_free(self.h)
            self.h = None
