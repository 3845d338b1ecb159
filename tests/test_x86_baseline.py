"""The timed CPU baseline (oracle/x86_graph_baseline.c: dequantise once, then per (sequence, head)
GEMV -> scale -> softmax -> GEMV in fp32) against the correctness oracle and against its own numpy twin."""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def xb():
    name = "x86_graph_baseline"
    if name not in sys.modules:
        spec = importlib.util.spec_from_file_location(name, ROOT / "oracle" / "x86_graph_baseline.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules[name]


def _case(rng, kv, Hq, Hkv, Dh, layout, num_layer=1):
    from ppl_nn_b200 import workloads
    idx = workloads.make_index(kv, [])
    cshape, sshape = workloads.cache_shapes(layout, idx.max_tokens, num_layer, Hkv, Dh)
    cache = rng.integers(-127, 128, size=cshape, dtype=np.int8)
    scale = rng.uniform(0.001, 0.0078, size=sshape).astype(np.float16)  # |values| < 1: fp16 half-ulp <= 2.5e-4
    q = rng.standard_normal((len(kv), Hq, Dh), dtype=np.float32).astype(np.float16)
    return idx, cache, scale, q


@pytest.mark.parametrize("Hq,Hkv,Dh", [(8, 8, 64), (8, 2, 128), (16, 2, 128)])
def test_baseline_matches_the_oracle_and_its_numpy_twin(xb, orc, pkg, Hq, Hkv, Dh):
    rng = np.random.default_rng(7)
    kv = np.array([1, 17, 64, 130, 255, 700], dtype=np.int64)
    idx, cache, scale, q = _case(rng, kv, Hq, Hkv, Dh, 0)
    base = xb.X86GraphBaseline(native=False, threads=4)
    st = base.prepare(Hkv, Dh, kv, idx.cachestarts, cache, scale)
    base.dequant(st)
    got = base.attention(st, q).astype(np.float64)
    twin = xb.np_attention(q, kv, idx.cachestarts, cache, scale)
    assert np.abs(got - twin).max() <= 1e-3  # one fp16 rounding of outputs of magnitude <= 1
    # the oracle of record reads the same cache through its own attention (no append: the cache is complete)
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, decoding_batches=idx.batch,
                 max_tokens=idx.max_tokens)
    want = orc.attention(d, q, np.zeros((len(kv), Hkv, Dh), np.float16), np.zeros((len(kv), Hkv, Dh), np.float16),
                         idx.seqstarts, idx.cachestarts, idx.start_pos, cache, scale).astype(np.float64)
    err = np.abs(got - want)
    assert err.max() <= 2e-3 and err.mean() <= 1e-4


def test_baseline_reads_layout_3_and_inner_layers(xb, pkg):
    rng = np.random.default_rng(8)
    kv = np.array([33, 5, 190], dtype=np.int64)
    Hq, Hkv, Dh, L, l = 8, 4, 64, 3, 1
    idx, cache0, scale0, q = _case(rng, kv, Hq, Hkv, Dh, 0, num_layer=L)
    base = xb.X86GraphBaseline(native=False, threads=2)
    st = base.prepare(Hkv, Dh, kv, idx.cachestarts, cache0, scale0, num_layer=L, layer_idx=l)
    base.dequant(st)
    a = base.attention(st, q)
    # the same contents in layout 3: (MaxT, L, 2, H, D) -> (L, 2, H, MaxT, D)
    cache3 = np.ascontiguousarray(cache0.transpose(1, 2, 3, 0, 4))
    scale3 = np.ascontiguousarray(scale0.transpose(1, 2, 3, 0, 4))
    st3 = base.prepare(Hkv, Dh, kv, idx.cachestarts, cache3, scale3, num_layer=L, layer_idx=l, cache_layout=3)
    base.dequant(st3)
    b = base.attention(st3, q)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    twin = xb.np_attention(q, kv, idx.cachestarts, np.ascontiguousarray(cache0[:, l:l + 1]),
                           np.ascontiguousarray(scale0[:, l:l + 1]))
    assert np.abs(a.astype(np.float64) - twin).max() <= 1e-3


def test_thread_count_is_set_explicitly(xb, monkeypatch):
    """A launcher's OMP_NUM_THREADS=1 must not silently turn the baseline into a one-thread run."""
    monkeypatch.setenv("OMP_NUM_THREADS", "1")
    base = xb.X86GraphBaseline(native=False, threads=3)
    assert base.num_threads() == 3
