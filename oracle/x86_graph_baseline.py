"""Python face of oracle/x86_graph_baseline.c.  TEST AND BENCHMARK INFRASTRUCTURE ONLY.

The C file restates, for decode sequences, the graph ppl.nn's x86 engine would run for this
mathematics -- per sequence ``MatMul(Q, K^T) -> Mul -> Softmax -> MatMul(P, V)`` in fp32 over the
already dequantised cache (src/ppl/nn/engines/x86/kernels/onnx/matmul_kernel.cc:45-52,
softmax_kernel.cc:41-51, OpenMP threading src/ppl/nn/engines/x86/threading.cc:24-26).  It is the
timed CPU baseline of the benchmark; the correctness oracle stays kvattn_oracle.c, and
``np_attention`` below is a numpy twin used to check the C file in the CPU tests.

Two builds: ``portable`` (x86-64-v3, travels between machines, used by the tests) and ``native``
(``-march=native``, rebuilt on the machine that times it).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "x86_graph_baseline.c"
_OUT_DIR = _HERE / "_build"


def _lib_path(native: bool) -> Path:
    return _OUT_DIR / ("libx86_graph_baseline.native.so" if native else "libx86_graph_baseline.so")


def build(native: bool = False, force: bool = False) -> Path:
    """Compile the C file.  The native build is always redone (it must match the host it runs on)."""
    out = _lib_path(native)
    if not native and out.exists() and not force and out.stat().st_mtime >= _SRC.stat().st_mtime:
        return out
    _OUT_DIR.mkdir(exist_ok=True)
    tmp = out.with_suffix(f".tmp{os.getpid()}")
    cmd = ["gcc", "-O3", "-march=native" if native else "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-Wall",
           "-Wextra", "-o", str(tmp), str(_SRC), "-lm"]
    subprocess.run(cmd, check=True)
    os.replace(tmp, out)
    return out


def host_threads() -> int:
    """Hardware threads this process may run on."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


class X86GraphBaseline:
    def __init__(self, native: bool = False, threads: int | None = None):
        self.lib = ctypes.CDLL(str(build(native=native)))
        L, vp, i32, i64 = self.lib, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
        L.xgb_dequant.restype = ctypes.c_int
        L.xgb_dequant.argtypes = [i32, i32, i32, i32, i32, i64, i64] + [vp] * 7
        L.xgb_attention.restype = ctypes.c_int
        L.xgb_attention.argtypes = [i32, i32, i32, i64] + [vp] * 6 + [i64, vp]
        L.xgb_num_threads.restype = ctypes.c_int
        L.xgb_set_num_threads.argtypes = [ctypes.c_int]
        L.xgb_set_num_threads.restype = None
        # a launcher may have exported OMP_NUM_THREADS=1; the baseline uses every thread it may run on
        L.xgb_set_num_threads(int(threads or host_threads()))

    def num_threads(self) -> int:
        return int(self.lib.xgb_num_threads())

    def prepare(self, num_kv_heads, head_dim, kvlens, cachestarts, cache, scale, *, num_layer=1, layer_idx=0,
                cache_layout=0, max_tokens=None):
        """Allocate the dense fp32 K/V matrices of a batch of decode sequences.  Returns a state dict for
        dequant() / attention()."""
        kvlens = np.ascontiguousarray(kvlens, dtype=np.int64)
        mat_starts = np.concatenate([[0], np.cumsum(kvlens * num_kv_heads)]).astype(np.int64)
        rows = int(mat_starts[-1])
        if max_tokens is None:
            max_tokens = cache.shape[0] if cache_layout == 0 else cache.shape[3]
        return dict(Hkv=int(num_kv_heads), Dh=int(head_dim), L=int(num_layer), l=int(layer_idx), layout=int(cache_layout),
                    max_tokens=int(max_tokens), kvlens=kvlens,
                    cachestarts=np.ascontiguousarray(cachestarts, dtype=np.int64), mat_starts=mat_starts,
                    cache=cache, scale=scale, K=np.empty((rows, head_dim), dtype=np.float32),
                    V=np.empty((rows, head_dim), dtype=np.float32),
                    scores=np.empty(self.num_threads() * max(int(kvlens.max()) if kvlens.size else 1, 1),
                                    dtype=np.float32))

    def dequant(self, st) -> None:
        rc = self.lib.xgb_dequant(st["Hkv"], st["Dh"], st["L"], st["l"], st["layout"], st["max_tokens"],
                                  st["kvlens"].size, _p(st["kvlens"]), _p(st["cachestarts"]), _p(st["mat_starts"]),
                                  _p(st["cache"]), _p(st["scale"]), _p(st["K"]), _p(st["V"]))
        if rc != 0:
            raise RuntimeError("xgb_dequant failed")

    def attention(self, st, query: np.ndarray, out: np.ndarray | None = None) -> np.ndarray:
        """query: float16 [batch, num_heads, head_dim] (one token per sequence)."""
        B, Hq, Dh = query.shape
        if out is None:
            out = np.empty((B, Hq, Dh), dtype=np.float16)
        rc = self.lib.xgb_attention(Hq, st["Hkv"], Dh, B, _p(st["kvlens"]), _p(st["mat_starts"]), _p(query),
                                    _p(st["K"]), _p(st["V"]), _p(st["scores"]),
                                    st["scores"].size // self.num_threads(), _p(out))
        if rc != 0:
            raise RuntimeError("xgb_attention failed")
        return out


def np_attention(query, kvlens, cachestarts, cache, scale):
    """numpy twin for layout 0, one layer: float64 attention over the dequantised rows."""
    B, Hq, Dh = query.shape
    Hkv = cache.shape[3]
    group = Hq // Hkv
    out = np.empty((B, Hq, Dh), dtype=np.float64)
    for b in range(B):
        rows = slice(int(cachestarts[b]), int(cachestarts[b] + kvlens[b]))
        deq = cache[rows, 0].astype(np.float64).reshape(-1, 2, Hkv, Dh // 8, 8) * \
            scale[rows, 0].astype(np.float64)[..., None]
        deq = deq.reshape(-1, 2, Hkv, Dh)
        for h in range(Hq):
            k, v = deq[:, 0, h // group], deq[:, 1, h // group]
            s = k @ query[b, h].astype(np.float64) / np.sqrt(Dh)
            p = np.exp(s - s.max())
            out[b, h] = (p / p.sum()) @ v
    return out
