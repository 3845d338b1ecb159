"""opmx.dynamic_batching.RotaryPositionEmbedding: oracle against its numpy twin and against properties of
a rotation (CPU); the CUDA kernel against the oracle, and the kernel fused with the cache append against
the two operators run one after the other (GPU).  Contract:
src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/rotary_position_embedding_kernel.cc:24-132."""
import struct

import numpy as np
import pytest

SCALINGS = [("", 1.0), ("linear", 4.0), ("dynamic", 2.0)]
CODE = {"": 0, "linear": 1, "dynamic": 2}


def _fbits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def _case(rng, seqlens, start_pos, Hq, Hkv, Dh):
    ss = np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int64)
    sp = np.asarray(start_pos, dtype=np.int64)
    q = rng.standard_normal((int(ss[-1]), Hq, Dh)).astype(np.float16)
    k = rng.standard_normal((int(ss[-1]), Hkv, Dh)).astype(np.float16)
    return q, k, ss, sp


# ---------------------------------------------------------------------------------------------------
# CPU
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("scaling,factor", SCALINGS)
@pytest.mark.parametrize("rotary_dim", [0, 32])
def test_c_oracle_equals_numpy_twin(orc, oracle_mod, scaling, factor, rotary_dim):
    rng = np.random.default_rng(3)
    q, k, ss, sp = _case(rng, [3, 1, 5, 2], [0, 4000, 100, 2047], 4, 2, 64)
    kw = dict(theta=10000.0, rotary_dim=rotary_dim, scaling_type=CODE[scaling], scaling_factor=factor,
              max_position_embeddings=2048)
    rq, rk = orc.rope(q, k, ss, sp, **kw)
    tq, tk = oracle_mod.np_rope(q, ss, sp, **kw), oracle_mod.np_rope(k, ss, sp, **kw)
    for got, want in ((rq, tq), (rk, tk)):
        diff = np.abs(got.astype(np.float32) - want.astype(np.float32))
        assert diff.max() <= 2 ** -8 and (diff > 0).mean() < 1e-3  # the twin's sin/cos may differ in the last bit
    if rotary_dim:
        np.testing.assert_array_equal(rq[..., rotary_dim:], q[..., rotary_dim:])  # pass-through channels


def test_rotation_properties(orc):
    rng = np.random.default_rng(4)
    q, k, ss, sp = _case(rng, [4, 4], [0, 7], 2, 2, 64)
    rq, rk = orc.rope(q, k, ss, sp, theta=10000.0)
    np.testing.assert_array_equal(rq[0], q[0])  # position 0: the identity
    # a rotation keeps the norm of every pair (up to fp16 rounding)
    n0 = np.hypot(q[..., 0::2].astype(np.float32), q[..., 1::2].astype(np.float32))
    n1 = np.hypot(rq[..., 0::2].astype(np.float32), rq[..., 1::2].astype(np.float32))
    assert np.abs(n0 - n1).max() < 4e-3
    # relative property: q(m).k(n) depends on m - n only -> same tokens shifted by 7 give the same scores
    s0 = np.einsum("ihd,jhd->hij", rq[0:4].astype(np.float32), rk[0:4].astype(np.float32))
    q2, k2 = np.concatenate([q[0:4], q[0:4]]), np.concatenate([k[0:4], k[0:4]])
    rq2, rk2 = orc.rope(q2, k2, ss, sp, theta=10000.0)
    s1 = np.einsum("ihd,jhd->hij", rq2[4:8].astype(np.float32), rk2[4:8].astype(np.float32))
    assert np.abs(s0 - s1).max() < 0.05
    # bypass_key leaves the key alone
    _, rkb = orc.rope(q, k, ss, sp, theta=10000.0, bypass_key=True)
    np.testing.assert_array_equal(rkb, k)


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


def test_theta_is_required_and_scaling_type_is_checked(host, engine):
    with pytest.raises(host.RetCodeError) as e:
        host.Op(engine, "RotaryPositionEmbedding", dict(rotary_dim=0))
    assert e.value.name == "RC_NOT_FOUND"
    with pytest.raises(host.RetCodeError) as e:
        host.Op(engine, "RotaryPositionEmbedding", dict(theta=_fbits(10000.0), scaling_type=3))
    assert e.value.name == "RC_UNSUPPORTED"
    host.Op(engine, "RotaryPositionEmbedding", dict(theta=_fbits(10000.0))).close()


def _fake(host, shape, dtype, on_host=False):
    t, _ = host.describe(np.zeros(shape, dtype=dtype))
    if not on_host:
        t.on_host = 0
        t.data = 4096  # never dereferenced on the paths tested
    return t


def test_kernel_guards(host, engine):
    op = host.Op(engine, "RotaryPositionEmbedding", dict(theta=_fbits(10000.0)))
    ms = np.array(4, dtype=np.int64)
    full = [_fake(host, (6, 8, 128), np.float16), _fake(host, (6, 2, 128), np.float16), _fake(host, (3,), np.int64),
            _fake(host, (2,), np.int64), host.describe(ms)[0]]
    outs = [_fake(host, (6, 8, 128), np.float16), _fake(host, (6, 2, 128), np.float16)]
    assert op.run_raw(full[:4], outs)[0] == "RC_NOT_FOUND"      # max_seqlen missing
    assert op.run_raw(full, outs[:1])[0] == "RC_NOT_FOUND"      # rotated_key missing
    bad = list(full)
    bad[0] = _fake(host, (6, 8, 128), np.float32)
    assert op.run_raw(bad, outs)[0] == "RC_UNSUPPORTED"         # fp16 only
    bad = list(full)
    bad[3] = _fake(host, (2,), np.int64, on_host=True)
    assert op.run_raw(bad, outs)[0] == "RC_INVALID_VALUE"       # start_pos on the host


# ---------------------------------------------------------------------------------------------------
# GPU
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def dev(built_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    assert built_lib.device_ready()
    d = torch.device("cuda:0")
    torch.cuda.set_device(d)
    return d


def _close(got, want):
    """Equal up to one fp16 unit in a handful of elements (device and host sin/cos differ in the last bit)."""
    g, w = got.astype(np.float32), want.astype(np.float32)
    diff = np.abs(g - w)
    assert diff.max() <= 2 ** -8, diff.max()          # one fp16 ulp at |x| in [2, 4)
    assert (diff > 0).mean() < 2e-3, (diff > 0).mean()


@pytest.mark.gpu
@pytest.mark.parametrize("scaling,factor", SCALINGS)
@pytest.mark.parametrize("Hq,Hkv,Dh,rotary_dim,bypass", [(8, 2, 128, 0, False), (4, 4, 64, 32, False), (8, 1, 128, 64, True)])
def test_gpu_matches_oracle(orc, dev, pkg, scaling, factor, Hq, Hkv, Dh, rotary_dim, bypass):
    import torch
    from ppl_nn_b200 import ops
    rng = np.random.default_rng(8)
    q, k, ss, sp = _case(rng, [70, 1, 1, 300, 5], [0, 4095, 130000, 1900, 17], Hq, Hkv, Dh)
    want_q, want_k = orc.rope(q, k, ss, sp, theta=500000.0, rotary_dim=rotary_dim, bypass_key=bypass,
                              scaling_type=CODE[scaling], scaling_factor=factor, max_position_embeddings=2048)
    op = ops.RotaryPositionEmbedding(ops.RotaryPositionEmbeddingParam(
        theta=500000.0, rotary_dim=rotary_dim, bypass_key=int(bypass), scaling_type=scaling, scaling_factor=factor,
        max_position_embeddings=2048))
    t = lambda a: torch.from_numpy(a).to(dev)
    rq, rk = op.forward(t(q), t(k), t(ss), t(sp), 300)
    _close(rq.cpu().numpy(), want_q)
    _close(rk.cpu().numpy(), want_k)
    # in place, as the reference does when it is the inputs' last consumer
    tq, tk = t(q), t(k)
    op.forward(tq, tk, t(ss), t(sp), 300, rotated_query=tq, rotated_key=tk)
    np.testing.assert_array_equal(tq.cpu().numpy().view(np.uint16), rq.cpu().numpy().view(np.uint16))
    np.testing.assert_array_equal(tk.cpu().numpy().view(np.uint16), rk.cpu().numpy().view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("pfl", [[70, 33], [700, 500]], ids=["one-kernel", "two-kernels"])
@pytest.mark.parametrize("mode,layout", [(0, 0), (0, 3), (1, 0)])
def test_fused_append_is_bit_identical_to_the_two_operators(orc, dev, pkg, mode, layout, pfl):
    import torch
    from ppl_nn_b200 import capi, ops, workloads
    rng = np.random.default_rng(9)
    Hq, Hkv, Dh, page = 8, 2, 128, 16
    kvl = [40, 17, 300]  # below 1024 tokens the call is one kernel, from there on two
    idx = workloads.make_index(kvl, pfl, page_size=page if mode else 0)
    T = idx.total_tokens
    q = rng.standard_normal((T, Hq, Dh)).astype(np.float16)
    k = rng.standard_normal((T, Hkv, Dh)).astype(np.float16)
    v = rng.standard_normal((T, Hkv, Dh)).astype(np.float16)
    cshape, sshape = workloads.cache_shapes(layout, idx.max_tokens, 1, Hkv, Dh)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    rope = ops.RotaryPositionEmbedding(ops.RotaryPositionEmbeddingParam(theta=10000.0))
    mk = lambda: ops.MultiHeadCacheAttention(ops.MultiHeadCacheAttentionParam(
        num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, num_layer=1, layer_idx=0, quant_bit=8, cache_mode=mode,
        cache_layout=layout, page_size=page))
    args_idx = (t(idx.seqstarts), t(idx.kvstarts), t(idx.cachestarts), t(idx.start_pos))
    # the two operators one after the other
    c1, s1 = torch.zeros(cshape, dtype=torch.int8, device=dev), torch.zeros(sshape, dtype=torch.float16, device=dev)
    rq, rk = rope.forward(t(q), t(k), args_idx[0], args_idx[3], idx.max_seqlen)
    a1 = mk()
    out1 = a1.forward(rq, rk, t(v), *args_idx, idx.decoding_batches, idx.max_seqlen, idx.max_kvlen, c1, s1)
    # fused rotation + append, then attention without its append phase
    c2, s2 = torch.zeros(cshape, dtype=torch.int8, device=dev), torch.zeros(sshape, dtype=torch.float16, device=dev)
    a2 = mk()
    rq2, rk2 = rope.forward_fused(a2, t(q), t(k), t(v), args_idx[0], args_idx[2], args_idx[3], idx.max_seqlen, c2, s2)
    out2 = a2.forward(rq2, rk2, t(v), *args_idx, idx.decoding_batches, idx.max_seqlen, idx.max_kvlen, c2, s2,
                      phase_mask=capi.PHASE_DECODE | capi.PHASE_PREFILL)
    assert a1.device_status() == 0 and a2.device_status() == 0
    np.testing.assert_array_equal(c1.cpu().numpy(), c2.cpu().numpy())
    np.testing.assert_array_equal(s1.cpu().numpy().view(np.uint16), s2.cpu().numpy().view(np.uint16))
    np.testing.assert_array_equal(rq.cpu().numpy().view(np.uint16), rq2.cpu().numpy().view(np.uint16))
    np.testing.assert_array_equal(rk.cpu().numpy().view(np.uint16), rk2.cpu().numpy().view(np.uint16))
    np.testing.assert_array_equal(out1.cpu().numpy().view(np.uint16), out2.cpu().numpy().view(np.uint16))
    # and the rotated key need not be written at all when nothing reads it
    rq3, rk3 = rope.forward_fused(mk(), t(q), t(k), t(v), args_idx[0], args_idx[2], args_idx[3], idx.max_seqlen,
                                  torch.zeros_like(c2), torch.zeros_like(s2), want_rotated_key=False)
    assert rk3 is None


@pytest.mark.gpu
def test_gpu_host_operator(orc, dev, pkg, host):
    import torch
    rng = np.random.default_rng(10)
    q, k, ss, sp = _case(rng, [9, 1, 40], [0, 77, 3], 8, 2, 128)
    want_q, want_k = orc.rope(q, k, ss, sp, theta=10000.0, scaling_type=1, scaling_factor=2.0)
    eng = host.Engine(0, torch.cuda.current_stream().cuda_stream)
    op = host.Op(eng, "RotaryPositionEmbedding", dict(theta=_fbits(10000.0), scaling_type=1, scaling_factor=_fbits(2.0)))
    t = lambda a: torch.from_numpy(a).to(dev)
    rq = torch.empty(q.shape, dtype=torch.float16, device=dev)
    rk = torch.empty(k.shape, dtype=torch.float16, device=dev)
    op.run([t(q), t(k), t(ss), t(sp), 40], [rq, rk])
    eng.synchronize()
    _close(rq.cpu().numpy(), want_q)
    _close(rk.cpu().numpy(), want_k)
    op.close()
    eng.close()


@pytest.mark.gpu
def test_host_operator_hands_input_buffers_over_when_it_is_their_last_consumer(orc, dev, pkg, host):
    """rotary_position_embedding_kernel.cc:55-75: as the last consumer of query / key the kernel moves their
    buffers to rotated_query / rotated_key (TransferBufferFrom) and rotates in place; otherwise the outputs get
    buffers of their own."""
    import torch
    rng = np.random.default_rng(12)
    q, k, ss, sp = _case(rng, [9, 1, 40], [0, 77, 3], 8, 2, 128)
    want_q, want_k = orc.rope(q, k, ss, sp, theta=10000.0)
    eng = host.Engine(0, torch.cuda.current_stream().cuda_stream)
    op = host.Op(eng, "RotaryPositionEmbedding", dict(theta=_fbits(10000.0)))
    t = lambda a: torch.from_numpy(a).to(dev)
    dq, dk = t(q), t(k)
    op.set_last_consumer(0)  # query only: rotated_query takes query's buffer, rotated_key is allocated
    res = op.run([dq, dk, t(ss), t(sp), 40], [None, None])
    eng.synchronize()
    assert res[0].data == dq.data_ptr() and res[1].data not in (None, 0, dk.data_ptr())
    _close(dq.cpu().numpy(), want_q)                      # rotated in place
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), k.view(np.uint16))  # key untouched
    dq2, dk2 = t(q), t(k)
    op.set_last_consumer(0, 1)
    res = op.run([dq2, dk2, t(ss), t(sp), 40], [None, None])
    eng.synchronize()
    assert res[0].data == dq2.data_ptr() and res[1].data == dk2.data_ptr()
    _close(dq2.cpu().numpy(), want_q)
    _close(dk2.cpu().numpy(), want_k)
    op.close()
    eng.close()
