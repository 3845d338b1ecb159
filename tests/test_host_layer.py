"""The C++ host layer (ppl.nn_b200/host) without a GPU: registry semantics, attribute parsing with
the reference's required/default attributes, engine knobs, and every guard of the two kernels that
is decided before any CUDA work.  Expected return codes follow the reference
(src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/*.cc, macros.h:84-89,
utils/op_info_manager.h:49-108)."""
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent

MHCA_ATTRS = dict(num_heads=8, num_kv_heads=2, head_dim=128, num_layer=2, layer_idx=1, quant_bit=8)
KVC_ATTRS = dict(num_layer=2, layer_idx=1, quant_bit=8)


@pytest.fixture(scope="module")
def host(built_lib, pkg):
    from ppl_nn_b200 import hostapi
    hostapi.register_ops()
    return hostapi


@pytest.fixture()
def engine(host):
    e = host.Engine(0, None)
    yield e
    e.close()


def test_host_header_symbols_are_exported(built_lib, host):
    header = (ROOT / "include" / "ppl_nn_b200_host.h").read_text()
    declared = set(re.findall(r"\b(pplb200_host_[a-z0-9_]+)\s*\(", header))
    assert declared == set(host.HOST_EXPORTS)
    for name in declared:
        assert hasattr(built_lib.dll, name), name


def test_registry_serves_the_reference_op_names(host):
    # register_ops.cc: ("opmx.dynamic_batching", "KeyValueCache" / "MultiHeadCacheAttention" / "MultiHeadAttention", 1, 1)
    assert host.registry_has("MultiHeadCacheAttention", 1)
    assert host.registry_has("KeyValueCache", 1)
    assert host.registry_has("MultiHeadAttention", 1)
    assert not host.registry_has("MultiHeadCacheAttention", 2)
    assert host.registry_has("RotaryPositionEmbedding", 1)
    assert not host.registry_has("ColumnParallelLinear", 1)
    assert not host.registry_has("MultiHeadCacheAttention", 1, domain="opmx")


def test_registry_register_overlap_remove(host):
    assert host.registry_register_again("MultiHeadCacheAttention", 1, 1) == "RC_EXISTS"
    assert host.registry_register_again("MultiHeadCacheAttention", 0, 3) == "RC_EXISTS"
    assert host.registry_register_again("MultiHeadCacheAttention", 2, 4) == "RC_SUCCESS"
    assert host.registry_has("MultiHeadCacheAttention", 3)
    assert host.registry_register_again("MultiHeadCacheAttention", 4, 5) == "RC_EXISTS"
    assert host.registry_register_again("MultiHeadCacheAttention", 5, 4) == "RC_INVALID_VALUE"
    host.registry_remove("MultiHeadCacheAttention")
    assert not host.registry_has("MultiHeadCacheAttention", 1)
    host.register_ops()  # Remove + Register: the documented way to swap an implementation in
    assert host.registry_has("MultiHeadCacheAttention", 1) and not host.registry_has("MultiHeadCacheAttention", 3)


@pytest.mark.parametrize("missing", ["num_heads", "head_dim", "num_layer", "layer_idx"])
def test_mhca_required_attributes(host, engine, missing):
    attrs = {k: v for k, v in MHCA_ATTRS.items() if k != missing}
    with pytest.raises(host.RetCodeError) as e:
        host.Op(engine, "MultiHeadCacheAttention", attrs)
    assert e.value.name == "RC_NOT_FOUND"


@pytest.mark.parametrize("missing", ["num_layer", "layer_idx"])
def test_kvcache_required_attributes(host, engine, missing):
    attrs = {k: v for k, v in KVC_ATTRS.items() if k != missing}
    with pytest.raises(host.RetCodeError) as e:
        host.Op(engine, "KeyValueCache", attrs)
    assert e.value.name == "RC_NOT_FOUND"


def test_unknown_op_is_not_found(host, engine):
    with pytest.raises(host.RetCodeError) as e:
        host.Op(engine, "ColumnParallelLinear", dict(num_layer=1, layer_idx=0))
    assert e.value.name == "RC_NOT_FOUND"


def test_engine_knobs(engine):
    assert engine.configure("cache_prefill", 1) == "RC_SUCCESS"
    assert engine.configure("decoding_attn_split_k", 2) == "RC_SUCCESS"
    assert engine.configure("decoding_attn_split_k", 3) == "RC_INVALID_VALUE"
    assert engine.configure("decoding_attn_tpb", 512) == "RC_SUCCESS"
    assert engine.configure("decoding_attn_tpb", 128) == "RC_INVALID_VALUE"
    for k in ("decoding_shm_mha", "decoding_inf_mha", "decoding_inf_gqa"):
        assert engine.configure(k, 0) == "RC_SUCCESS"
    assert engine.configure("graph_fusion", 1) == "RC_INVALID_VALUE"


# ---- kernel guards that need no GPU ----------------------------------------------------------------
def _mhca_inputs(host, *, T=4, B=4, Hq=8, Hkv=2, Dh=128, L=2, maxt=64, fake=4096, drop_after=None, scale=True,
                 attn_mask=None, mask_dtype=np.float16, cachestarts_2d=False, q_dtype=np.float16):
    """HostTensor structs with fake device pointers: nothing below dereferences them on the paths tested."""
    def dev(shape, dtype):
        t, _ = host.describe(np.zeros(shape, dtype=dtype))
        t.on_host = 0
        t.data = fake
        return t
    ins = [dev((T, Hq, Dh), q_dtype), dev((T, Hkv, Dh), np.float16), dev((T, Hkv, Dh), np.float16),
           dev((B + 1,), np.int64), dev((B + 1,), np.int64),
           dev((B, 4) if cachestarts_2d else (B,), np.int64), dev((B,), np.int64)]
    keep = [np.array(B, dtype=np.int64), np.array(1, dtype=np.int64), np.array(32, dtype=np.int64)]
    for k in keep:
        ins.append(host.describe(k)[0])
    ins.append(dev((maxt, L, 2, Hkv, Dh), np.int8))
    if scale is True:
        ins.append(dev((maxt, L, 2, Hkv, Dh // 8), np.float16))
    elif scale == "empty":
        ins.append(dev((0,), np.float16))
    elif scale is None:
        ins.append(host.describe(None)[0])
    if attn_mask is not None:
        ins.append(dev(attn_mask, mask_dtype))
    if drop_after is not None:
        ins = ins[:drop_after]
    out = dev((T, Hq, Dh), np.float16)
    return ins, [out], keep


@pytest.mark.parametrize("n_inputs,name", [(10, "cache"), (6, "start_pos"), (0, "query")])
def test_mhca_missing_required_input(host, engine, n_inputs, name):
    op = host.Op(engine, "MultiHeadCacheAttention", MHCA_ATTRS)
    ins, outs, keep = _mhca_inputs(host, drop_after=n_inputs)
    rc, _ = op.run_raw(ins, outs)
    assert rc == "RC_NOT_FOUND"


def test_mhca_missing_output(host, engine):
    op = host.Op(engine, "MultiHeadCacheAttention", MHCA_ATTRS)
    ins, outs, keep = _mhca_inputs(host)
    rc, _ = op.run_raw(ins, [])
    assert rc == "RC_NOT_FOUND"


@pytest.mark.parametrize("attrs,kw,expect", [
    (dict(quant_bit=4), {}, "RC_UNSUPPORTED"),
    (dict(quant_group=16), {}, "RC_UNSUPPORTED"),
    (dict(quant_bit=0), {}, "RC_UNSUPPORTED"),          # the parser default: an unquantised cache is not supported
    (dict(is_alibi=1), {}, "RC_UNSUPPORTED"),
    ({}, dict(scale=None), "RC_UNSUPPORTED"),
    ({}, dict(scale="empty"), "RC_UNSUPPORTED"),
    ({}, dict(attn_mask=(4, 8), mask_dtype=np.float32), "RC_UNSUPPORTED"),  # the mask is fp16
    ({}, dict(attn_mask=(5,)), "RC_INVALID_VALUE"),       # [T, C] or [num_heads, T, C]
    ({}, dict(attn_mask=(4, 4)), "RC_INVALID_VALUE"),     # C must be a multiple of 8
    ({}, dict(attn_mask=(2, 8)), "RC_INVALID_VALUE"),     # fewer rows than query tokens
    ({}, dict(attn_mask=(3, 4, 8)), "RC_INVALID_VALUE"),  # leading dimension is not num_heads
    ({}, dict(q_dtype=np.float32), "RC_UNSUPPORTED"),
    (dict(cache_layout=1), {}, "RC_UNSUPPORTED"),
    (dict(cache_mode=1), {}, "RC_INVALID_VALUE"),        # paged mode with 1-d cachestarts
])
def test_mhca_guards(host, engine, attrs, kw, expect):
    op = host.Op(engine, "MultiHeadCacheAttention", {**MHCA_ATTRS, **attrs})
    ins, outs, keep = _mhca_inputs(host, **kw)
    rc, _ = op.run_raw(ins, outs)
    assert rc == expect


@pytest.mark.parametrize("which,shape,dtype", [
    (0, (4, 8, 64), np.float16),      # query with another head_dim than the attribute
    (0, (4, 1024), np.float16),       # query flattened to 2-d
    (1, (4, 4, 128), np.float16),     # current_key with another head count
    (2, (3, 2, 128), np.float16),     # current_value with fewer tokens than query
    (3, (4,), np.int64),              # seqstarts shorter than batch + 1
    (4, (5,), np.int32),              # kvstarts not int64
    (5, (3,), np.int64),              # cachestarts shorter than batch
    (10, (64 * 2, 2, 2, 128), np.int8),  # cache not 5-d
])
def test_mhca_rejects_tensors_the_kernels_would_overrun(host, engine, which, shape, dtype):
    op = host.Op(engine, "MultiHeadCacheAttention", MHCA_ATTRS)
    ins, outs, keep = _mhca_inputs(host)
    t, _ = host.describe(np.zeros(shape, dtype=dtype))
    t.on_host = 0
    t.data = 4096
    ins[which] = t
    rc, _ = op.run_raw(ins, outs)
    assert rc == "RC_INVALID_VALUE"


def test_bound_call_gives_the_same_return_codes(host, engine):
    """Op.bind builds the argument arrays once; its call() must behave like run_raw on the same structs."""
    for attrs, expect in ((dict(cache_layout=1), "RC_UNSUPPORTED"), (dict(cache_mode=1), "RC_INVALID_VALUE")):
        op = host.Op(engine, "MultiHeadCacheAttention", {**MHCA_ATTRS, **attrs})
        ins, outs, keep = _mhca_inputs(host)
        call, bound_outs = op.bind(ins, outs)
        assert call() == expect == op.run_raw(ins, outs)[0]
        assert call() == expect  # and again, with the same arrays
        assert list(bound_outs[0].dims[:3]) == [4, 8, 128]  # Reshape ran: attn_output took query's shape


def test_mhca_empty_attn_mask_counts_as_absent_and_output_takes_query_shape(host, engine):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this case passes every guard; with a GPU it would launch kernels on the fake pointers")
    op = host.Op(engine, "MultiHeadCacheAttention", MHCA_ATTRS)
    ins, outs, keep = _mhca_inputs(host, attn_mask=(0,))  # zero elements: absent
    outs[0].ndim = 1
    outs[0].dims[0] = 7  # stale shape: Reshape must overwrite it with query's
    rc, res = op.run_raw(ins, outs)
    # all guards passed; without a GPU the tmp-buffer allocation is where the call stops
    assert rc == "RC_OUT_OF_MEMORY"
    assert res[0].ndim == 3 and list(res[0].dims[:3]) == [4, 8, 128] and res[0].dtype == host.DT_FLOAT16


def test_kvcache_shape_inference_and_guards(host, engine):
    op = host.Op(engine, "KeyValueCache", KVC_ATTRS)

    def dev(shape, dtype, data=4096):
        t, _ = host.describe(np.zeros(shape, dtype=dtype))
        t.on_host = 0
        t.data = data
        return t

    kvstarts = np.array([0, 5, 9, 30], dtype=np.int64)  # host tensor: the op reads kvstarts[-1] from its device
    ks, _ = host.describe(kvstarts)
    base = [dev((3, 2, 128), np.float16), dev((3, 2, 128), np.float16), dev((4,), np.int64), ks, dev((3,), np.int64),
            dev((3,), np.int64), host.describe(1)[0], host.describe(30)[0], dev((64, 2, 2, 2, 128), np.int8)]
    outs = [dev((1,), np.float16), dev((1,), np.float16)]
    # scale missing -> RC_UNSUPPORTED, but the outputs were already reshaped to [kvstarts[-1], Hkv, Dh]
    rc, res = op.run_raw(base, outs)
    assert rc == "RC_UNSUPPORTED"
    assert [list(r.dims[:3]) for r in res] == [[30, 2, 128], [30, 2, 128]]
    # kvstarts without a buffer: outputs get length 0 and the kernel reports RC_NOT_FOUND
    nobuf = list(base)
    nobuf[3], _ = host.describe(kvstarts, no_buffer=True)
    rc, res = op.run_raw(nobuf + [dev((64, 2, 2, 2, 16), np.float16)], outs)
    assert rc == "RC_NOT_FOUND" and list(res[0].dims[:3]) == [0, 2, 128]
    # num_repeat != 1
    op2 = host.Op(engine, "KeyValueCache", {**KVC_ATTRS, "num_repeat": 2})
    rc, _ = op2.run_raw(base + [dev((64, 2, 2, 2, 16), np.float16)], outs)
    assert rc == "RC_UNSUPPORTED"
    # fewer inputs than the contract
    rc, _ = op.run_raw(base[:5], outs)
    assert rc == "RC_NOT_FOUND"
