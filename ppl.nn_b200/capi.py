"""ctypes binding of the C ABI declared in include/ppl_nn_b200.h.

Only pointers and integers cross this boundary.  The library is loaded from ``lib/`` next to this
file and never falls back to anything else: if it is missing, or was built without sm_100a code for
the current device, the calls fail with an error.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import os

HERE = Path(__file__).resolve().parent
# PPLB200_LIBRARY selects another build of the same library (kernel tuning experiments)
LIB_PATH = Path(os.environ["PPLB200_LIBRARY"]) if os.environ.get("PPLB200_LIBRARY") else HERE / "lib" / "libppl_nn_b200.so"

SUCCESS = 0
INVALID_VALUE = 1
UNSUPPORTED = 2
OUT_OF_MEMORY = 3
DEVICE_RUNTIME_ERROR = 4
NOT_FOUND = 5
NO_DEVICE_CODE = 6

PHASE_APPEND = 1
PHASE_DECODE = 2
PHASE_PREFILL = 4

DEV_OK = 0
DEV_TMA_WAIT_TIMEOUT = 1
DEV_MMA_WAIT_TIMEOUT = 2
DEV_LENGTH_CLAMPED = 4
DEV_ROW_OUT_OF_RANGE = 8
DEV_MASK_OUT_OF_RANGE = 16

# every symbol include/ppl_nn_b200.h declares
EXPORTS = (
    "pplb200_fill_cache_strides",
    "pplb200_kv_append_i8g8",
    "pplb200_kv_gather_dequant",
    "pplb200_mhca_workspace_size",
    "pplb200_mhca_forward",
    "pplb200_mhca_forward_masked",
    "pplb200_attn_mask_check",
    "pplb200_mhca_forward_noalloc",
    "pplb200_static_scratch_bytes",
    "pplb200_static_scratch_status",
    "pplb200_mhca_device_status",
    "pplb200_mha_workspace_size",
    "pplb200_mha_forward",
    "pplb200_mha_forward_masked",
    "pplb200_rope_workspace_size",
    "pplb200_rope_forward",
    "pplb200_rope_kv_append_i8g8",
    "pplb200_status_str",
    "pplb200_device_ready",
    "pplb200_launch_count",
    "pplb200_profile_enable",
    "pplb200_profile_read",
)

KERNEL_APPEND = 0
KERNEL_DECODE = 1
KERNEL_PREFILL = 2


class AttnParams(ctypes.Structure):
    """Mirror of ``pplb200_attn_params``; field order and types must match the header."""

    _fields_ = [
        ("num_heads", ctypes.c_int32), ("num_kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("is_causal", ctypes.c_int32), ("num_layer", ctypes.c_int32), ("layer_idx", ctypes.c_int32),
        ("quant_bit", ctypes.c_int32), ("quant_group", ctypes.c_int32), ("cache_mode", ctypes.c_int32),
        ("cache_layout", ctypes.c_int32), ("page_size", ctypes.c_int32),
        ("enable_cache_prefill", ctypes.c_int32), ("split_k_mode", ctypes.c_int32), ("phase_mask", ctypes.c_int32),
        ("batch", ctypes.c_int64), ("decoding_batches", ctypes.c_int64), ("max_seqlen", ctypes.c_int64),
        ("max_kvlen", ctypes.c_int64), ("total_tokens", ctypes.c_int64), ("max_tokens", ctypes.c_int64),
        ("cache_stride_s", ctypes.c_int64), ("cache_stride_l", ctypes.c_int64), ("cache_stride_h", ctypes.c_int64),
        ("cache_stride_kv", ctypes.c_int64), ("cachestart_stride_b", ctypes.c_int64),
    ]

    def copy(self) -> "AttnParams":
        other = AttnParams()
        ctypes.memmove(ctypes.byref(other), ctypes.byref(self), ctypes.sizeof(self))
        return other


class MhaParams(ctypes.Structure):
    """Mirror of ``pplb200_mha_params``."""

    _fields_ = [
        ("num_heads", ctypes.c_int32), ("num_kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("is_causal", ctypes.c_int32),
        ("batch", ctypes.c_int64), ("decoding_batches", ctypes.c_int64), ("max_seqlen", ctypes.c_int64),
        ("max_kvlen", ctypes.c_int64), ("total_tokens", ctypes.c_int64), ("total_kv_tokens", ctypes.c_int64),
    ]


class AttnMask(ctypes.Structure):
    """Mirror of ``pplb200_attn_mask``: the optional additive fp16 mask, [T, C] or [num_heads, T, C]."""

    _fields_ = [("data", ctypes.c_void_p), ("ndim", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("dims", ctypes.c_int64 * 3)]

    @classmethod
    def of(cls, data_ptr: int, shape) -> "AttnMask":
        m = cls()
        m.data = data_ptr
        m.ndim = len(shape)
        for i, d in enumerate(shape[:3]):
            m.dims[i] = int(d)
        return m


class RopeParams(ctypes.Structure):
    """Mirror of ``pplb200_rope_params``."""

    _fields_ = [
        ("num_heads", ctypes.c_int32), ("num_kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("rotary_dim", ctypes.c_int32), ("bypass_key", ctypes.c_int32), ("scaling_type", ctypes.c_int32),
        ("max_position_embeddings", ctypes.c_int32), ("reserved", ctypes.c_int32),
        ("theta", ctypes.c_float), ("scaling_factor", ctypes.c_float),
        ("batch", ctypes.c_int64), ("max_seqlen", ctypes.c_int64), ("total_tokens", ctypes.c_int64),
    ]


class StatusError(RuntimeError):
    def __init__(self, fn: str, code: int, name: str):
        super().__init__(f"{fn} returned {name} ({code})")
        self.code = code
        self.name = name


class Library:
    """The loaded shared library with typed entry points."""

    def __init__(self, path: Path | str | None = None):
        p = Path(path) if path else LIB_PATH
        if not p.exists():
            raise FileNotFoundError(
                f"{p} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(there is no CPU or PyTorch fallback for these operators)")
        self.path = p
        self.dll = ctypes.CDLL(str(p))
        d = self.dll
        vp, i64p = ctypes.c_void_p, ctypes.c_void_p
        pp = ctypes.POINTER(AttnParams)
        d.pplb200_fill_cache_strides.restype = ctypes.c_int
        d.pplb200_fill_cache_strides.argtypes = [pp]
        d.pplb200_kv_append_i8g8.restype = ctypes.c_int
        d.pplb200_kv_append_i8g8.argtypes = [pp, vp, vp, i64p, i64p, i64p, vp, vp, vp]
        d.pplb200_kv_gather_dequant.restype = ctypes.c_int
        d.pplb200_kv_gather_dequant.argtypes = [pp, i64p, i64p, vp, vp, ctypes.c_int64, vp, vp, vp]
        d.pplb200_mhca_workspace_size.restype = ctypes.c_int
        d.pplb200_mhca_workspace_size.argtypes = [pp, ctypes.POINTER(ctypes.c_uint64)]
        d.pplb200_mhca_forward.restype = ctypes.c_int
        d.pplb200_mhca_forward.argtypes = [pp, vp, vp, vp, i64p, i64p, i64p, i64p, vp, vp, vp, ctypes.c_uint64, vp, vp]
        kp = ctypes.POINTER(AttnMask)
        d.pplb200_mhca_forward_masked.restype = ctypes.c_int
        d.pplb200_mhca_forward_masked.argtypes = [pp, vp, vp, vp, i64p, i64p, i64p, i64p, vp, vp, kp, vp,
                                                  ctypes.c_uint64, vp, vp]
        d.pplb200_mhca_forward_noalloc.restype = ctypes.c_int
        d.pplb200_mhca_forward_noalloc.argtypes = [pp, vp, vp, vp, i64p, i64p, i64p, i64p, vp, vp, vp, vp]
        d.pplb200_static_scratch_bytes.restype = ctypes.c_uint64
        d.pplb200_static_scratch_bytes.argtypes = []
        d.pplb200_static_scratch_status.restype = ctypes.c_int
        d.pplb200_static_scratch_status.argtypes = [vp, ctypes.POINTER(ctypes.c_uint32)]
        d.pplb200_mhca_device_status.restype = ctypes.c_int
        d.pplb200_mhca_device_status.argtypes = [vp, vp, ctypes.POINTER(ctypes.c_uint32)]
        mp = ctypes.POINTER(MhaParams)
        d.pplb200_mha_workspace_size.restype = ctypes.c_int
        d.pplb200_mha_workspace_size.argtypes = [mp, ctypes.POINTER(ctypes.c_uint64)]
        d.pplb200_mha_forward.restype = ctypes.c_int
        d.pplb200_mha_forward.argtypes = [mp, vp, vp, vp, i64p, i64p, vp, ctypes.c_uint64, vp, vp]
        d.pplb200_mha_forward_masked.restype = ctypes.c_int
        d.pplb200_mha_forward_masked.argtypes = [mp, vp, vp, vp, i64p, i64p, kp, vp, ctypes.c_uint64, vp, vp]
        rp = ctypes.POINTER(RopeParams)
        d.pplb200_rope_workspace_size.restype = ctypes.c_int
        d.pplb200_rope_workspace_size.argtypes = [rp, ctypes.POINTER(ctypes.c_uint64)]
        d.pplb200_rope_forward.restype = ctypes.c_int
        d.pplb200_rope_forward.argtypes = [rp, vp, vp, i64p, i64p, vp, ctypes.c_uint64, vp, vp, vp]
        d.pplb200_rope_kv_append_i8g8.restype = ctypes.c_int
        d.pplb200_rope_kv_append_i8g8.argtypes = [rp, pp, vp, vp, vp, i64p, i64p, i64p, vp, ctypes.c_uint64, vp, vp,
                                                  vp, vp, vp]
        d.pplb200_status_str.restype = ctypes.c_char_p
        d.pplb200_status_str.argtypes = [ctypes.c_int]
        d.pplb200_device_ready.restype = ctypes.c_int
        d.pplb200_device_ready.argtypes = []
        d.pplb200_launch_count.restype = ctypes.c_uint64
        d.pplb200_launch_count.argtypes = []
        d.pplb200_profile_enable.restype = ctypes.c_int
        d.pplb200_profile_enable.argtypes = [ctypes.c_int]
        d.pplb200_profile_read.restype = ctypes.c_int
        d.pplb200_profile_read.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double),
                                           ctypes.POINTER(ctypes.c_uint64)]

    # ---- helpers ------------------------------------------------------------------------
    def status_str(self, code: int) -> str:
        return self.dll.pplb200_status_str(int(code)).decode()

    def check(self, fn: str, code: int) -> None:
        if code != SUCCESS:
            raise StatusError(fn, code, self.status_str(code))

    def device_ready(self) -> bool:
        return bool(self.dll.pplb200_device_ready())

    def launch_count(self) -> int:
        return int(self.dll.pplb200_launch_count())

    def profile_enable(self, on: bool) -> None:
        self.check("pplb200_profile_enable", self.dll.pplb200_profile_enable(1 if on else 0))

    def profile_read(self, family: int) -> tuple[float, int]:
        """(summed device milliseconds, launches) of one kernel family since the last read."""
        ms, n = ctypes.c_double(0), ctypes.c_uint64(0)
        self.check("pplb200_profile_read", self.dll.pplb200_profile_read(family, ctypes.byref(ms), ctypes.byref(n)))
        return float(ms.value), int(n.value)

    # ---- raw entry points: return the status code -----------------------------------------
    def fill_cache_strides(self, p: AttnParams) -> int:
        return self.dll.pplb200_fill_cache_strides(ctypes.byref(p))

    def kv_append(self, p, cur_k, cur_v, seqstarts, cachestarts, start_pos, cache, scale, stream) -> int:
        return self.dll.pplb200_kv_append_i8g8(ctypes.byref(p), cur_k, cur_v, seqstarts, cachestarts, start_pos,
                                               cache, scale, stream)

    def kv_gather_dequant(self, p, kvstarts, cachestarts, cache, scale, total_kv, key_out, value_out, stream) -> int:
        return self.dll.pplb200_kv_gather_dequant(ctypes.byref(p), kvstarts, cachestarts, cache, scale,
                                                  int(total_kv), key_out, value_out, stream)

    def mhca_workspace_size(self, p) -> tuple[int, int]:
        n = ctypes.c_uint64(0)
        rc = self.dll.pplb200_mhca_workspace_size(ctypes.byref(p), ctypes.byref(n))
        return rc, int(n.value)

    def mhca_forward(self, p, q, cur_k, cur_v, seqstarts, kvstarts, cachestarts, start_pos, cache, scale,
                     workspace, workspace_bytes, out, stream) -> int:
        return self.dll.pplb200_mhca_forward(ctypes.byref(p), q, cur_k, cur_v, seqstarts, kvstarts, cachestarts,
                                             start_pos, cache, scale, workspace, int(workspace_bytes), out, stream)

    def mhca_forward_masked(self, p, q, cur_k, cur_v, seqstarts, kvstarts, cachestarts, start_pos, cache, scale,
                            mask: "AttnMask | None", workspace, workspace_bytes, out, stream) -> int:
        return self.dll.pplb200_mhca_forward_masked(ctypes.byref(p), q, cur_k, cur_v, seqstarts, kvstarts, cachestarts,
                                                    start_pos, cache, scale,
                                                    ctypes.byref(mask) if mask is not None else None, workspace,
                                                    int(workspace_bytes), out, stream)

    def mha_forward_masked(self, p, q, k, v, seqstarts, kvstarts, mask: "AttnMask | None", workspace,
                           workspace_bytes, out, stream) -> int:
        return self.dll.pplb200_mha_forward_masked(ctypes.byref(p), q, k, v, seqstarts, kvstarts,
                                                   ctypes.byref(mask) if mask is not None else None, workspace,
                                                   int(workspace_bytes), out, stream)

    def static_scratch_status(self, stream) -> tuple[int, int]:
        """Device status word the last no-alloc call left in the built-in scratch (synchronises the stream)."""
        s = ctypes.c_uint32(0)
        rc = self.dll.pplb200_static_scratch_status(stream, ctypes.byref(s))
        return rc, int(s.value)

    def mhca_forward_noalloc(self, p, q, cur_k, cur_v, seqstarts, kvstarts, cachestarts, start_pos, cache, scale,
                             out, stream) -> int:
        """Same as mhca_forward but with the library's built-in scratch: no workspace, no allocation."""
        return self.dll.pplb200_mhca_forward_noalloc(ctypes.byref(p), q, cur_k, cur_v, seqstarts, kvstarts,
                                                     cachestarts, start_pos, cache, scale, out, stream)

    def mha_workspace_size(self, p) -> tuple[int, int]:
        n = ctypes.c_uint64(0)
        rc = self.dll.pplb200_mha_workspace_size(ctypes.byref(p), ctypes.byref(n))
        return rc, int(n.value)

    def mha_forward(self, p, q, k, v, seqstarts, kvstarts, workspace, workspace_bytes, out, stream) -> int:
        return self.dll.pplb200_mha_forward(ctypes.byref(p), q, k, v, seqstarts, kvstarts, workspace,
                                            int(workspace_bytes), out, stream)

    def rope_workspace_size(self, p) -> tuple[int, int]:
        n = ctypes.c_uint64(0)
        rc = self.dll.pplb200_rope_workspace_size(ctypes.byref(p), ctypes.byref(n))
        return rc, int(n.value)

    def rope_forward(self, p, q, k, seqstarts, start_pos, workspace, workspace_bytes, rq, rk, stream) -> int:
        return self.dll.pplb200_rope_forward(ctypes.byref(p), q, k, seqstarts, start_pos, workspace,
                                             int(workspace_bytes), rq, rk, stream)

    def rope_kv_append(self, p, attn, q, k, v, seqstarts, cachestarts, start_pos, workspace, workspace_bytes, rq, rk,
                       cache, scale, stream) -> int:
        return self.dll.pplb200_rope_kv_append_i8g8(ctypes.byref(p), ctypes.byref(attn), q, k, v, seqstarts,
                                                    cachestarts, start_pos, workspace, int(workspace_bytes), rq, rk,
                                                    cache, scale, stream)

    def static_scratch_bytes(self) -> int:
        return int(self.dll.pplb200_static_scratch_bytes())

    def mhca_device_status(self, workspace, stream) -> tuple[int, int]:
        s = ctypes.c_uint32(0)
        rc = self.dll.pplb200_mhca_device_status(workspace, stream, ctypes.byref(s))
        return rc, int(s.value)


_LIB: Library | None = None


def library() -> Library:
    global _LIB
    if _LIB is None:
        _LIB = Library()
    return _LIB
