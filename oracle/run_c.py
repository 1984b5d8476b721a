"""CPU ORACLE runner — test infrastructure only.

Compiles the C text printed by `oracle.emit_c` with the cc backend's own
command line (`cc <file.c> -O3 -march=native -o <lib.so> -shared -fPIC`,
arrayjit/lib/cc_backend.ml:77-101; no -ffast-math, :21,:90), loads it and
calls the routine with numpy buffers in the sorted-parameter order of
`C_syntax.compile_proc` (arrayjit/lib/c_syntax.ml:1080-1084), the way
`Cc_backend.link_compiled` builds its call (cc_backend.ml:378-443).
Runs on one host thread, as the reference's `sync_cc` does
(arrayjit/lib/schedulers.ml:284).

One flag is added to that command line: `-fno-tree-loop-if-convert`.  gcc 13.3 with
`-O3 -march=native` on an AVX-512 host (preferred vector width 256) miscompiles the
vectorised form of `(y[i] > 0.0 ? (y[i] - t[i]) * (float)(0.5) : 0.0)` — the C spelling of a
relu gate over single-precision nodes, a float value selected in a double comparison — and
reads zeros or stale lanes in place of `t` for the upper half of each 16-element row; the
same text gives the right values at -O0, -O2, -O3 without -march, and with if-conversion or
loop vectorisation off.  A checker must not depend on that, so if-conversion is off here;
the contraction loops, which carry the run time, are not affected by it.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import time
from typing import Dict, Optional

import numpy as np

from .emit_c import Emitter

_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, "_build")

NP_DTYPE = {"byte": np.uint8, "uint16": np.uint16, "int32": np.int32, "uint32": np.uint32,
            "int64": np.int64, "uint64": np.uint64, "half": np.float16, "bfloat16": np.uint16,
            "fp8": np.uint8, "single": np.float32, "double": np.float64,
            # four 32-bit words per element: arrays of this precision get a trailing axis of 4
            "uint4x32": np.dtype((np.uint32, (4,)))}


class OracleRoutine:
    def __init__(self, ir_text: str, cc: str = "gcc"):
        self.em = Emitter(ir_text)
        self.src = self.em.source()
        os.makedirs(_BUILD, exist_ok=True)
        tag = hashlib.sha256((self.src + "|no-if-convert").encode()).hexdigest()[:20]
        self.c_path = os.path.join(_BUILD, "%s_%s.c" % (self.em.name, tag))
        self.so_path = self.c_path[:-2] + ".so"
        if not os.path.exists(self.so_path):
            with open(self.c_path, "w") as f:
                f.write(self.src)
            tmp = self.so_path + ".tmp%d" % os.getpid()
            subprocess.run([cc, self.c_path, "-O3", "-march=native", "-fno-tree-loop-if-convert", "-o", tmp,
                            "-shared", "-fPIC", "-I", _HERE, "-lm"], check=True)
            os.replace(tmp, self.so_path)
        self.lib = ctypes.CDLL(self.so_path)
        self.fn = getattr(self.lib, self.em.name)
        self.fn.restype = None
        self.params = self.em.params()

    def buffers(self) -> Dict[str, np.ndarray]:
        """Zero-filled numpy buffers for every parameter node, keyed by ident."""
        out = {}
        for _, (kind, ref) in self.params:
            if kind == "tn":
                t = self.em.tn[ref]
                out[t["ident"]] = np.zeros(t["dims"] if t["dims"] else [1], NP_DTYPE[t["prec"]])
        return out

    def run(self, bufs: Dict[str, np.ndarray], static: Optional[Dict[str, int]] = None,
            merge: Optional[np.ndarray] = None) -> float:
        """Calls the routine in place on `bufs`; returns the wall time in seconds."""
        args = []
        for _, (kind, ref) in self.params:
            if kind == "tn":
                a = bufs[self.em.tn[ref]["ident"]]
                assert a.flags["C_CONTIGUOUS"]
                args.append(ctypes.c_void_p(a.ctypes.data))
            elif kind == "static":
                args.append(ctypes.c_uint32(int((static or {})[ref])))
            else:
                args.append(ctypes.c_void_p(merge.ctypes.data))
        t0 = time.perf_counter()
        self.fn(*args)
        return time.perf_counter() - t0
