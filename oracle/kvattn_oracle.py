"""Python face of the CPU oracle.  TEST INFRASTRUCTURE ONLY -- PARITY UNPINNED.

Two independent restatements of the same contract live here:

* ``CORacle`` loads ``kvattn_oracle.c`` (compiled by :func:`build`) through ctypes.  It is the
  oracle of record for the tests, the smoke check and the benchmark's CPU baseline.
* ``np_quant_groups`` / ``np_dequant`` / ``np_attention_one`` are a numpy twin of the same formulas,
  written separately so that the C file is itself checked (the two must agree bit for bit on
  the quantiser and to fp32 round-off on attention).

Neither is ever imported by the CUDA product path.  "Parity unpinned" means: the reference
tree (ppl.nn) contains no source, test or golden vector for the arithmetic of this path -- it
lives in the un-vendored ppl.llm.kernel.cuda module -- so the quantisation formula below is the
one fixed by this repository from the published description "INT8 symmetric groupwise, group 8,
fp16 scale = absmax / 127", not one verified against the reference's own output.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "kvattn_oracle.c"
_OUT_DIR = _HERE / "_build"
_LIB = _OUT_DIR / "libkvattn_oracle.so"


def build(force: bool = False) -> Path:
    """Compile kvattn_oracle.c into oracle/_build/ (x86-64-v3 so the file runs on any recent host)."""
    if _LIB.exists() and not force and _LIB.stat().st_mtime >= _SRC.stat().st_mtime:
        return _LIB
    _OUT_DIR.mkdir(exist_ok=True)
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-Wall", "-Wextra",
           "-o", str(_LIB), str(_SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


class OrcDesc(ctypes.Structure):
    _fields_ = [
        ("num_heads", ctypes.c_int32), ("num_kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("is_causal", ctypes.c_int32), ("num_layer", ctypes.c_int32), ("layer_idx", ctypes.c_int32),
        ("quant_group", ctypes.c_int32), ("cache_mode", ctypes.c_int32), ("cache_layout", ctypes.c_int32),
        ("page_size", ctypes.c_int32), ("enable_cache_prefill", ctypes.c_int32), ("reserved", ctypes.c_int32),
        ("batch", ctypes.c_int64), ("decoding_batches", ctypes.c_int64), ("max_tokens", ctypes.c_int64),
        ("cachestart_stride_b", ctypes.c_int64),
    ]


class OrcMask(ctypes.Structure):
    """The optional attn_mask input: additive fp16, [T, C] or [num_heads, T, C] (see orc_mask in the C file)."""
    _fields_ = [("data", ctypes.c_void_p), ("heads", ctypes.c_int64), ("rows", ctypes.c_int64), ("cols", ctypes.c_int64)]


def _mask(m: np.ndarray | None):
    if m is None or m.size == 0:
        return None
    assert m.dtype == np.float16 and m.flags["C_CONTIGUOUS"] and m.ndim in (2, 3)
    heads = m.shape[0] if m.ndim == 3 else 1
    return OrcMask(m.ctypes.data, heads, m.shape[-2], m.shape[-1])


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ctypes.c_void_p)


class COracle:
    """ctypes wrapper over the compiled C oracle.  fp16 tensors are numpy float16 arrays."""

    def __init__(self, lib_path: os.PathLike | None = None):
        path = Path(lib_path) if lib_path else (_LIB if _LIB.exists() else build())
        self.lib = ctypes.CDLL(str(path))
        L = self.lib
        L.orc_half_to_float.restype = ctypes.c_float
        L.orc_half_to_float.argtypes = [ctypes.c_uint16]
        L.orc_float_to_half.restype = ctypes.c_uint16
        L.orc_float_to_half.argtypes = [ctypes.c_float]
        vp = ctypes.c_void_p
        L.orc_quant_group.restype = None
        L.orc_quant_group.argtypes = [vp, vp, vp]
        L.orc_kv_append.restype = ctypes.c_int
        L.orc_kv_append.argtypes = [ctypes.POINTER(OrcDesc)] + [vp] * 7
        L.orc_kv_gather_dequant.restype = ctypes.c_int
        L.orc_kv_gather_dequant.argtypes = [ctypes.POINTER(OrcDesc)] + [vp] * 6
        L.orc_attention.restype = ctypes.c_int
        L.orc_attention.argtypes = [ctypes.POINTER(OrcDesc)] + [vp] * 9 + [ctypes.c_int64, ctypes.c_int64]
        L.orc_mhca.restype = ctypes.c_int
        L.orc_mhca.argtypes = [ctypes.POINTER(OrcDesc)] + [vp] * 9
        L.orc_rope.restype = ctypes.c_int
        L.orc_rope.argtypes = [ctypes.c_int64] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_float,
                               ctypes.c_float, ctypes.c_int64] + [vp] * 6
        L.orc_mha.restype = ctypes.c_int
        L.orc_mha.argtypes = [ctypes.POINTER(OrcDesc)] + [vp] * 6
        L.orc_mhca_masked.restype = ctypes.c_int
        L.orc_mhca_masked.argtypes = [ctypes.POINTER(OrcDesc)] + [vp] * 10 + [ctypes.POINTER(OrcMask)]
        L.orc_mha_masked.restype = ctypes.c_int
        L.orc_mha_masked.argtypes = [ctypes.POINTER(OrcDesc)] + [vp] * 6 + [ctypes.POINTER(OrcMask)]
        L.orc_num_threads.restype = ctypes.c_int

    # -- scalar helpers ---------------------------------------------------------------
    def half_to_float(self, h: int) -> float:
        return float(self.lib.orc_half_to_float(h))

    def float_to_half(self, f: float) -> int:
        return int(self.lib.orc_float_to_half(ctypes.c_float(f)))

    def num_threads(self) -> int:
        return int(self.lib.orc_num_threads())

    def quant_groups(self, x: np.ndarray):
        """x: float16 [..., 8k] -> (int8 codes same shape, float16 scales [..., k])."""
        x = np.ascontiguousarray(x, dtype=np.float16)
        flat = x.reshape(-1, 8)
        codes = np.empty(flat.shape, dtype=np.int8)
        scales = np.empty(flat.shape[0], dtype=np.float16)
        for i in range(flat.shape[0]):
            self.lib.orc_quant_group(flat[i].ctypes.data_as(ctypes.c_void_p),
                                     codes[i].ctypes.data_as(ctypes.c_void_p),
                                     ctypes.c_void_p(scales.ctypes.data + 2 * i))
        return codes.reshape(x.shape), scales.reshape(x.shape[:-1] + (x.shape[-1] // 8,))

    # -- operators --------------------------------------------------------------------
    @staticmethod
    def desc(**kw) -> OrcDesc:
        d = OrcDesc()
        d.quant_group = 8
        d.page_size = 128
        d.num_layer = 1
        d.is_causal = 1
        for k, v in kw.items():
            if not hasattr(d, k):
                raise KeyError(k)
            setattr(d, k, int(v))
        return d

    def kv_append(self, d, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache, scale):
        rc = self.lib.orc_kv_append(ctypes.byref(d), _ptr(cur_k), _ptr(cur_v), _ptr(seqstarts), _ptr(cachestarts),
                                    _ptr(start_pos), _ptr(cache), _ptr(scale))
        if rc != 0:
            raise RuntimeError(f"orc_kv_append failed: {rc}")

    def kv_gather_dequant(self, d, kvstarts, cachestarts, cache, scale):
        total = int(kvstarts[-1])
        key = np.empty((total, d.num_kv_heads, d.head_dim), dtype=np.float16)
        value = np.empty_like(key)
        rc = self.lib.orc_kv_gather_dequant(ctypes.byref(d), _ptr(kvstarts), _ptr(cachestarts), _ptr(cache),
                                            _ptr(scale), _ptr(key), _ptr(value))
        if rc != 0:
            raise RuntimeError(f"orc_kv_gather_dequant failed: {rc}")
        return key, value

    def attention(self, d, query, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache, scale,
                  seq_lo: int = 0, seq_hi: int | None = None, out: np.ndarray | None = None):
        if out is None:
            out = np.zeros(query.shape, dtype=np.float16)
        hi = int(d.batch) if seq_hi is None else int(seq_hi)
        rc = self.lib.orc_attention(ctypes.byref(d), _ptr(query), _ptr(cur_k), _ptr(cur_v), _ptr(seqstarts),
                                    _ptr(cachestarts), _ptr(start_pos), _ptr(cache), _ptr(scale), _ptr(out),
                                    int(seq_lo), hi)
        if rc != 0:
            raise RuntimeError(f"orc_attention failed: {rc}")
        return out

    def mhca(self, d, query, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache, scale, *, kvstarts=None,
             attn_mask=None):
        """The whole operator: append, then attend.  `attn_mask` (with `kvstarts`): the optional additive mask."""
        out = np.zeros(query.shape, dtype=np.float16)
        m = _mask(attn_mask)
        if m is None:
            rc = self.lib.orc_mhca(ctypes.byref(d), _ptr(query), _ptr(cur_k), _ptr(cur_v), _ptr(seqstarts),
                                   _ptr(cachestarts), _ptr(start_pos), _ptr(cache), _ptr(scale), _ptr(out))
        else:
            rc = self.lib.orc_mhca_masked(ctypes.byref(d), _ptr(query), _ptr(cur_k), _ptr(cur_v), _ptr(seqstarts),
                                          _ptr(kvstarts), _ptr(cachestarts), _ptr(start_pos), _ptr(cache), _ptr(scale),
                                          _ptr(out), ctypes.byref(m))
        if rc != 0:
            raise RuntimeError(f"orc_mhca failed: {rc}")
        return out

    def mha(self, d, query, key, value, seqstarts, kvstarts, *, attn_mask=None):
        """The un-cached operator: attention over the call's own key/value tensors."""
        out = np.zeros(query.shape, dtype=np.float16)
        m = _mask(attn_mask)
        if m is None:
            rc = self.lib.orc_mha(ctypes.byref(d), _ptr(query), _ptr(key), _ptr(value), _ptr(seqstarts),
                                  _ptr(kvstarts), _ptr(out))
        else:
            rc = self.lib.orc_mha_masked(ctypes.byref(d), _ptr(query), _ptr(key), _ptr(value), _ptr(seqstarts),
                                         _ptr(kvstarts), _ptr(out), ctypes.byref(m))
        if rc != 0:
            raise RuntimeError(f"orc_mha failed: {rc}")
        return out

    def rope(self, query, key, seqstarts, start_pos, *, theta=10000.0, rotary_dim=0, bypass_key=False,
             scaling_type=0, scaling_factor=1.0, max_position_embeddings=2048):
        """RotaryPositionEmbedding: (rotated_query, rotated_key); scaling_type 0 none, 1 linear, 2 dynamic."""
        rq, rk = np.empty_like(query), np.empty_like(key)
        rc = self.lib.orc_rope(query.shape[1], key.shape[1], query.shape[2], int(rotary_dim), int(bool(bypass_key)),
                               int(scaling_type), int(max_position_embeddings), ctypes.c_float(theta),
                               ctypes.c_float(scaling_factor), len(start_pos), _ptr(query), _ptr(key), _ptr(seqstarts),
                               _ptr(start_pos), _ptr(rq), _ptr(rk))
        if rc != 0:
            raise RuntimeError(f"orc_rope failed: {rc}")
        return rq, rk


# ------------------------------------------------------------------ numpy twin ---------

def np_quant_groups(x: np.ndarray):
    """Same formula as orc_quant_group, vectorised.  x: float16 [..., 8k]."""
    x = np.asarray(x, dtype=np.float16)
    g = x.reshape(x.shape[:-1] + (x.shape[-1] // 8, 8)).astype(np.float32)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        a = np.fmax.reduce(np.abs(g), axis=-1, initial=np.float32(0))  # fmax ignores NaN like `m > a`
        s16 = (a / np.float32(127.0)).astype(np.float16)
        s = s16.astype(np.float32)[..., None]
        q = np.rint(g / s)  # numpy rint is round-half-to-even
        q = np.where(q >= -127.0, q, np.float32(-127.0))  # NaN -> -127 like the C code
        q = np.where(q > 127.0, np.float32(127.0), q)
        q = np.where(s != 0, q, np.float32(0))
    return q.astype(np.int8).reshape(x.shape), s16


def np_dequant(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """float32 dequantised values; codes [..., 8k] int8, scales [..., k] float16."""
    c = codes.reshape(codes.shape[:-1] + (codes.shape[-1] // 8, 8)).astype(np.float32)
    return (c * scales.astype(np.float32)[..., None]).reshape(codes.shape)


def np_attention_one(q: np.ndarray, k: np.ndarray, v: np.ndarray, mask_row: np.ndarray | None = None) -> np.ndarray:
    """One query vector against n_kv rows; all float32.  q [Dh], k/v [n_kv, Dh] -> [Dh]; `mask_row` [n_kv] is added
    to the scaled scores; a row masked with -inf everywhere gives zeros."""
    s = (k @ q) * np.float32(1.0 / np.sqrt(np.float32(q.shape[0])))
    if mask_row is not None:
        s = s + mask_row.astype(np.float32)
    if not s.max() > -np.inf:
        return np.zeros(v.shape[1], dtype=np.float32)
    p = np.exp(s - s.max())
    return (p @ v) / p.sum()


def np_mha(query, key, value, seqstarts, kvstarts, num_kv_heads: int, is_causal: bool, attn_mask=None) -> np.ndarray:
    """numpy twin of orc_mha (float32 inside, fp16 result): causal masks aligned to the end of the kv range;
    attn_mask [T, C] or [Hq, T, C] is indexed [.., seqstarts[b] + i, kvstarts[b] + j]."""
    T, Hq, Dh = query.shape
    group = Hq // num_kv_heads
    out = np.zeros((T, Hq, Dh), dtype=np.float16)
    q32, k32, v32 = (np.asarray(x, dtype=np.float32) for x in (query, key, value))
    for b in range(len(seqstarts) - 1):
        s0, s1, k0, k1 = int(seqstarts[b]), int(seqstarts[b + 1]), int(kvstarts[b]), int(kvstarts[b + 1])
        seqlen, kvlen = s1 - s0, k1 - k0
        for i in range(seqlen):
            n = min(kvlen, (kvlen - seqlen) + i + 1) if is_causal else kvlen
            if n <= 0:
                continue
            for h in range(Hq):
                kvh = h // group
                mrow = None
                if attn_mask is not None:
                    mrow = (attn_mask[h] if attn_mask.ndim == 3 else attn_mask)[s0 + i, k0:k0 + n]
                out[s0 + i, h] = np_attention_one(q32[s0 + i, h], k32[k0:k0 + n, kvh], v32[k0:k0 + n, kvh],
                                                  mrow).astype(np.float16)
    return out


def np_rope(x, seqstarts, start_pos, *, theta=10000.0, rotary_dim=0, scaling_type=0, scaling_factor=1.0,
            max_position_embeddings=2048) -> np.ndarray:
    """numpy twin of orc_rope for one tensor [T, H, Dh] (fp16 in and out)."""
    T, H, Dh = x.shape
    rot = Dh if rotary_dim == 0 else rotary_dim
    out = np.array(x, dtype=np.float16, copy=True)
    j = np.arange(rot // 2, dtype=np.float64)
    for b in range(len(start_pos)):
        s0, s1 = int(seqstarts[b]), int(seqstarts[b + 1])
        th = float(np.float32(theta))
        L = int(start_pos[b]) + (s1 - s0)
        if scaling_type == 2 and L > max_position_embeddings:
            f = float(np.float32(scaling_factor))
            th = th * (f * L / max_position_embeddings - (f - 1.0)) ** (rot / (rot - 2.0))
        inv = np.power(th, -2.0 * j / rot).astype(np.float32)
        pos = (np.arange(s1 - s0, dtype=np.int64) + int(start_pos[b])).astype(np.float32)
        if scaling_type == 1:
            pos = pos / np.float32(scaling_factor)
        ang = (pos[:, None] * inv[None, :]).astype(np.float32)
        sn, cs = np.sin(ang)[:, None, :], np.cos(ang)[:, None, :]
        x0 = x[s0:s1, :, 0:rot:2].astype(np.float32)
        x1 = x[s0:s1, :, 1:rot:2].astype(np.float32)
        out[s0:s1, :, 0:rot:2] = ((x0 * cs).astype(np.float32) - (x1 * sn).astype(np.float32)).astype(np.float16)
        out[s0:s1, :, 1:rot:2] = ((x0 * sn).astype(np.float32) + (x1 * cs).astype(np.float32)).astype(np.float16)
    return out
