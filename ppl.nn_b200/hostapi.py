"""ctypes face of the C++ host layer (include/ppl_nn_b200_host.h): the two operators created through
the llm_cuda-style registry and executed as engine kernels.  This is the reference-facing way to call
the path; ``ops.py`` is the thinner route that goes straight to the C ABI."""
from __future__ import annotations

import ctypes

import numpy as np

from . import capi

DT_FLOAT16, DT_FLOAT32, DT_INT8, DT_INT32, DT_INT64 = 1, 2, 3, 4, 5

HOST_EXPORTS = (
    "pplb200_host_engine_create", "pplb200_host_engine_destroy", "pplb200_host_engine_configure",
    "pplb200_host_engine_tmp_pool_bytes", "pplb200_host_register_ops", "pplb200_host_registry_has",
    "pplb200_host_registry_remove", "pplb200_host_registry_register_again", "pplb200_host_op_create",
    "pplb200_host_op_destroy", "pplb200_host_op_run", "pplb200_host_op_set_last_consumer",
    "pplb200_host_engine_synchronize",
    "pplb200_host_retcode_str",
)

DOMAIN = "opmx.dynamic_batching"


class HostTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("dims", ctypes.c_int64 * 6), ("on_host", ctypes.c_int32), ("absent", ctypes.c_int32)]


class RetCodeError(RuntimeError):
    def __init__(self, what: str, name: str):
        super().__init__(f"{what}: {name}")
        self.name = name


def _dll():
    d = capi.library().dll
    if getattr(d, "_host_typed", False):
        return d
    vp = ctypes.c_void_p
    d.pplb200_host_engine_create.restype = vp
    d.pplb200_host_engine_create.argtypes = [ctypes.c_int, vp]
    d.pplb200_host_engine_destroy.restype = None
    d.pplb200_host_engine_destroy.argtypes = [vp]
    d.pplb200_host_engine_configure.restype = ctypes.c_int
    d.pplb200_host_engine_configure.argtypes = [vp, ctypes.c_char_p, ctypes.c_int64]
    d.pplb200_host_engine_tmp_pool_bytes.restype = ctypes.c_uint64
    d.pplb200_host_engine_tmp_pool_bytes.argtypes = [vp]
    d.pplb200_host_register_ops.restype = None
    d.pplb200_host_register_ops.argtypes = []
    d.pplb200_host_registry_has.restype = ctypes.c_int
    d.pplb200_host_registry_has.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint64]
    d.pplb200_host_registry_remove.restype = None
    d.pplb200_host_registry_remove.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    d.pplb200_host_registry_register_again.restype = ctypes.c_int
    d.pplb200_host_registry_register_again.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint64]
    d.pplb200_host_op_create.restype = vp
    d.pplb200_host_op_create.argtypes = [vp, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint64,
                                         ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_int64), ctypes.c_int,
                                         ctypes.POINTER(ctypes.c_int)]
    d.pplb200_host_op_destroy.restype = None
    d.pplb200_host_op_destroy.argtypes = [vp]
    d.pplb200_host_op_run.restype = ctypes.c_int
    d.pplb200_host_op_run.argtypes = [vp, ctypes.POINTER(HostTensor), ctypes.c_int, ctypes.POINTER(HostTensor),
                                      ctypes.c_int]
    d.pplb200_host_op_set_last_consumer.restype = None
    d.pplb200_host_op_set_last_consumer.argtypes = [vp, ctypes.c_uint32]
    d.pplb200_host_engine_synchronize.restype = ctypes.c_int
    d.pplb200_host_engine_synchronize.argtypes = [vp]
    d.pplb200_host_retcode_str.restype = ctypes.c_char_p
    d.pplb200_host_retcode_str.argtypes = [ctypes.c_int]
    d._host_typed = True
    return d


def retcode_str(rc: int) -> str:
    return _dll().pplb200_host_retcode_str(int(rc)).decode()


def register_ops() -> None:
    _dll().pplb200_host_register_ops()


def registry_has(type_: str, version: int = 1, domain: str = DOMAIN) -> bool:
    return bool(_dll().pplb200_host_registry_has(domain.encode(), type_.encode(), version))


def registry_remove(type_: str, domain: str = DOMAIN) -> None:
    _dll().pplb200_host_registry_remove(domain.encode(), type_.encode())


def registry_register_again(type_: str, first: int, last: int, domain: str = DOMAIN) -> str:
    return retcode_str(_dll().pplb200_host_registry_register_again(domain.encode(), type_.encode(), first, last))


_NP_DT = {np.dtype(np.float16): DT_FLOAT16, np.dtype(np.float32): DT_FLOAT32, np.dtype(np.int8): DT_INT8,
          np.dtype(np.int32): DT_INT32, np.dtype(np.int64): DT_INT64}


def describe(x, *, absent: bool = False, no_buffer: bool = False) -> tuple[HostTensor, object]:
    """HostTensor for a torch tensor (device or host), a numpy array (host), an int (host int64 scalar),
    or None (an optional input that the graph leaves out).  Returns (struct, keep-alive object)."""
    t = HostTensor()
    if x is None or absent:
        t.absent = 1
        return t, None
    if isinstance(x, (int, np.integer)):
        x = np.array(int(x), dtype=np.int64)
    if isinstance(x, np.ndarray):
        x = np.ascontiguousarray(x)
        t.data = None if no_buffer else x.ctypes.data
        t.dtype = _NP_DT[x.dtype]
        t.on_host = 1
        shape = x.shape
    else:  # torch tensor
        import torch
        assert x.is_contiguous()
        t.data = None if no_buffer else x.data_ptr()
        t.dtype = {torch.float16: DT_FLOAT16, torch.float32: DT_FLOAT32, torch.int8: DT_INT8, torch.int32: DT_INT32,
                   torch.int64: DT_INT64}[x.dtype]
        t.on_host = 0 if x.is_cuda else 1
        shape = tuple(x.shape)
    t.ndim = len(shape)
    for i, d in enumerate(shape):
        t.dims[i] = d
    return t, x


class Engine:
    def __init__(self, device_id: int = 0, stream: int | None = None):
        self.d = _dll()
        self.handle = self.d.pplb200_host_engine_create(device_id, stream)
        if not self.handle:
            raise RuntimeError("pplb200_host_engine_create failed")

    def configure(self, key: str, value: int) -> str:
        return retcode_str(self.d.pplb200_host_engine_configure(self.handle, key.encode(), int(value)))

    def tmp_pool_bytes(self) -> int:
        return int(self.d.pplb200_host_engine_tmp_pool_bytes(self.handle))

    def synchronize(self) -> None:
        rc = self.d.pplb200_host_engine_synchronize(self.handle)
        if rc != 0:
            raise RetCodeError("synchronize", retcode_str(rc))

    def close(self):
        if self.handle:
            self.d.pplb200_host_engine_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Op:
    """An operator instance: node + attributes + Op + Kernel, created through the registry."""

    def __init__(self, engine: Engine, type_: str, attrs: dict, version: int = 1, domain: str = DOMAIN):
        self.engine = engine
        self.d = engine.d
        names = (ctypes.c_char_p * len(attrs))(*[k.encode() for k in attrs])
        values = (ctypes.c_int64 * len(attrs))(*[int(v) for v in attrs.values()])
        rc = ctypes.c_int(0)
        self.handle = self.d.pplb200_host_op_create(engine.handle, domain.encode(), type_.encode(), version, names,
                                                    values, len(attrs), ctypes.byref(rc))
        if not self.handle:
            raise RetCodeError(f"create {domain}:{type_}:{version}", retcode_str(rc.value))

    def set_last_consumer(self, *input_indices: int) -> None:
        """Tell the op that it is the last consumer of these inputs (what the runtime derives from the graph)."""
        mask = 0
        for i in input_indices:
            mask |= 1 << int(i)
        self.d.pplb200_host_op_set_last_consumer(self.handle, mask)

    def run_raw(self, inputs: list, outputs: list) -> tuple[str, list[HostTensor]]:
        """inputs/outputs: HostTensor structs.  Returns (RetCode name, output structs after the run)."""
        ins = (HostTensor * len(inputs))(*inputs)
        outs = (HostTensor * len(outputs))(*outputs)
        rc = self.d.pplb200_host_op_run(self.handle, ins, len(inputs), outs, len(outputs))
        return retcode_str(rc), list(outs)

    def bind(self, inputs: list, outputs: list):
        """For a loop that runs the operator on the same buffers every step: builds the argument arrays once
        and returns (call, output structs); call() runs the operator and returns the RetCode name."""
        ins = (HostTensor * len(inputs))(*inputs)
        outs = (HostTensor * len(outputs))(*outputs)
        run, handle, n_in, n_out = self.d.pplb200_host_op_run, self.handle, len(inputs), len(outputs)

        def call() -> str:
            rc = run(handle, ins, n_in, outs, n_out)
            return "RC_SUCCESS" if rc == 0 else retcode_str(rc)

        return call, outs

    def run(self, inputs: list, outputs: list):
        """inputs: torch tensors / numpy arrays / ints / None; outputs: torch tensors to write into, or
        None to let the kernel allocate.  Raises RetCodeError unless RC_SUCCESS."""
        keep = []
        ins = []
        for x in inputs:
            t, k = describe(x)
            ins.append(t)
            keep.append(k)
        outs = []
        for x in outputs:
            if x is None:
                t = HostTensor()
            else:
                t, k = describe(x)
                keep.append(k)
            outs.append(t)
        name, res = self.run_raw(ins, outs)
        if name != "RC_SUCCESS":
            raise RetCodeError("run", name)
        return res

    def close(self):
        if self.handle:
            self.d.pplb200_host_op_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
