"""opmx.dynamic_batching.MultiHeadAttention (attention over the call's own key/value tensors, no cache).
CPU part: the C oracle against its numpy twin, the attribute parser and the host kernel's guards
(src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/multi_head_attention_kernel.cc:24-128).
GPU part: the CUDA path against the oracle through the C ABI and through the host-layer operator."""
import numpy as np
import pytest

MAX_ABS = 2e-3
MEAN_ABS = 1e-3
MHA_ATTRS = dict(num_heads=8, num_kv_heads=2, head_dim=128)


def _case(rng, seqlens, kvlens, Hq, Hkv, Dh, scale=1.0):
    ss = np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int64)
    ks = np.concatenate([[0], np.cumsum(kvlens)]).astype(np.int64)
    q = (rng.standard_normal((int(ss[-1]), Hq, Dh)) * scale).astype(np.float16)
    k = (rng.standard_normal((max(int(ks[-1]), 1), Hkv, Dh)) * scale).astype(np.float16)[:int(ks[-1])]
    v = rng.standard_normal((max(int(ks[-1]), 1), Hkv, Dh)).astype(np.float16)[:int(ks[-1])]
    return q, k, v, ss, ks


# ---------------------------------------------------------------------------------------------------
# CPU
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("causal", [True, False])
def test_c_oracle_equals_numpy_twin(orc, oracle_mod, causal):
    rng = np.random.default_rng(11)
    q, k, v, ss, ks = _case(rng, [3, 1, 5, 4, 2], [7, 9, 5, 2, 0], 4, 2, 64)
    d = orc.desc(num_heads=4, num_kv_heads=2, head_dim=64, batch=5, is_causal=int(causal))
    got = orc.mha(d, q, k, v, ss, ks)
    want = oracle_mod.np_mha(q, k, v, ss, ks, 2, causal)
    np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), atol=2e-3, rtol=0)
    if causal:
        # sequence 3 has 4 query rows and 2 kv rows: the mask is aligned to the end, rows 0 and 1 see nothing
        assert not got[ss[3]:ss[3] + 2].any() and got[ss[3] + 2:ss[4]].any()
    assert not got[ss[4]:ss[5]].any()  # no kv rows at all: zeros


def test_causal_with_equal_lengths_is_the_prefill_of_the_cached_operator(orc):
    """kvlen == seqlen, causal: the same numbers as the cached operator's prefill over current_key/value."""
    rng = np.random.default_rng(12)
    Hq, Hkv, Dh = 4, 2, 64
    q, k, v, ss, ks = _case(rng, [5, 9], [5, 9], Hq, Hkv, Dh)
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=2, is_causal=1)
    a = orc.mha(d, q, k, v, ss, ks)
    d2 = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=2, decoding_batches=0, max_tokens=16)
    cache = np.zeros((16, 1, 2, Hkv, Dh), dtype=np.int8)
    scale = np.zeros((16, 1, 2, Hkv, Dh // 8), dtype=np.float16)
    b = orc.mhca(d2, q, k, v, ss, np.array([0, 5], dtype=np.int64), np.zeros(2, dtype=np.int64), cache, scale)
    np.testing.assert_array_equal(a.view(np.uint16), b.view(np.uint16))


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


@pytest.mark.parametrize("missing", ["num_heads", "head_dim"])
def test_required_attributes(host, engine, missing):
    attrs = {k: v for k, v in MHA_ATTRS.items() if k != missing}
    with pytest.raises(host.RetCodeError) as e:
        host.Op(engine, "MultiHeadAttention", attrs)
    assert e.value.name == "RC_NOT_FOUND"


def _fake_inputs(host, *, T=6, Tkv=9, B=2, Hq=8, Hkv=2, Dh=128, drop_after=None, attn_mask=None,
                 mask_dtype=np.float16, q_dtype=np.float16):
    def dev(shape, dtype):
        t, _ = host.describe(np.zeros(shape, dtype=dtype))
        t.on_host = 0
        t.data = 4096  # never dereferenced on the paths tested
        return t
    ins = [dev((T, Hq, Dh), q_dtype), dev((Tkv, Hkv, Dh), np.float16), dev((Tkv, Hkv, Dh), np.float16),
           dev((B + 1,), np.int64), dev((B + 1,), np.int64)]
    keep = [np.array(0, dtype=np.int64), np.array(4, dtype=np.int64), np.array(8, dtype=np.int64)]
    for k in keep:
        ins.append(host.describe(k)[0])
    if attn_mask is not None:
        ins.append(dev(attn_mask, mask_dtype))
    if drop_after is not None:
        ins = ins[:drop_after]
    return ins, [dev((T, Hq, Dh), np.float16)], keep


@pytest.mark.parametrize("n_inputs", [7, 4, 0])
def test_missing_required_input(host, engine, n_inputs):
    op = host.Op(engine, "MultiHeadAttention", MHA_ATTRS)
    ins, outs, keep = _fake_inputs(host, drop_after=n_inputs)
    assert op.run_raw(ins, outs)[0] == "RC_NOT_FOUND"


@pytest.mark.parametrize("attrs,kw,expect", [
    (dict(is_alibi=1), {}, "RC_UNSUPPORTED"),
    ({}, dict(q_dtype=np.float32), "RC_UNSUPPORTED"),
    ({}, dict(attn_mask=(6, 16), mask_dtype=np.float32), "RC_UNSUPPORTED"),  # the mask is fp16
    ({}, dict(attn_mask=(6, 9)), "RC_INVALID_VALUE"),      # columns must be a multiple of 8
    ({}, dict(attn_mask=(4, 16)), "RC_INVALID_VALUE"),     # fewer rows than query tokens
    ({}, dict(attn_mask=(3, 6, 16)), "RC_INVALID_VALUE"),  # leading dimension is not num_heads
])
def test_guards(host, engine, attrs, kw, expect):
    op = host.Op(engine, "MultiHeadAttention", {**MHA_ATTRS, **attrs})
    ins, outs, keep = _fake_inputs(host, **kw)
    assert op.run_raw(ins, outs)[0] == expect


def test_host_index_tensor_is_refused(host, engine):
    op = host.Op(engine, "MultiHeadAttention", MHA_ATTRS)
    ins, outs, keep = _fake_inputs(host)
    ins[3] = host.describe(np.zeros(3, dtype=np.int64))[0]  # seqstarts on the host
    assert op.run_raw(ins, outs)[0] == "RC_INVALID_VALUE"


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


CASES = [
    # seqlens, kvlens, Hq, Hkv, Dh
    ([40], [40], 8, 2, 128),
    ([1, 1, 1], [17, 64, 130], 8, 8, 64),                 # decode-like: one query row against fp16 history
    ([130, 7, 257, 64], [130, 7, 257, 64], 8, 2, 128),    # ragged, tile edges
    ([5, 128, 33], [69, 200, 33], 4, 1, 128),             # kv longer than q: mask aligned to the end
    ([9, 4], [3, 0], 4, 2, 64),                           # fewer kv rows than query rows, and none at all
    ([300], [1000], 32, 8, 128),
    ([300] * 40, [10] * 40, 4, 2, 128),                   # runs of query tiles that see no kv row at all
    # one-token sequences with several query heads per kv head: the heads of a group share one tile
    ([1] * 5, [17, 64, 130, 1, 300], 32, 4, 128),
    ([1, 1, 1], [70, 5, 129], 16, 8, 64),
    ([1, 1], [0, 9], 8, 2, 64),                           # ... and a sequence without any kv row
]


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("case", CASES, ids=[str(i) for i in range(len(CASES))])
def test_gpu_matches_oracle(orc, dev, pkg, case, causal):
    import torch
    from ppl_nn_b200 import ops
    seqlens, kvlens, Hq, Hkv, Dh = case
    rng = np.random.default_rng(100 + len(seqlens) + Hq)
    q, k, v, ss, ks = _case(rng, seqlens, kvlens, Hq, Hkv, Dh)
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=len(seqlens), is_causal=int(causal))
    want = orc.mha(d, q, k, v, ss, ks).astype(np.float32)
    op = ops.MultiHeadAttention(ops.MultiHeadAttentionParam(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, is_causal=causal))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    kk = k if k.shape[0] else np.zeros((1, Hkv, Dh), dtype=np.float16)
    vv = v if v.shape[0] else np.zeros((1, Hkv, Dh), dtype=np.float16)
    out = torch.full((q.shape[0], Hq, Dh), float("nan"), dtype=torch.float16, device=dev)
    got = op.forward(t(q), t(kk)[:k.shape[0]], t(vv)[:v.shape[0]], t(ss), t(ks), 0, max(seqlens), max(kvlens),
                     attn_output=out)
    assert op.device_status() == 0
    got = got.cpu().numpy().astype(np.float32)
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max(), err.mean())


def _mask_for(rng, q_rows, kv_rows, heads=None):
    C = (kv_rows + 7) // 8 * 8
    shape = (q_rows, C) if heads is None else (heads, q_rows, C)
    m = (rng.standard_normal(shape) * 0.5).astype(np.float16)
    m[rng.random(shape) < 0.2] = -np.inf
    return m


@pytest.mark.parametrize("per_head", [False, True])
def test_oracle_mask_matches_its_numpy_twin(orc, oracle_mod, per_head):
    """attn_mask in the C oracle against the numpy restatement: additive, [T, C] or [heads, T, C], element
    [.., seqstarts[b] + i, kvstarts[b] + j], on top of the causal mask; a fully removed row gives zeros."""
    rng = np.random.default_rng(17)
    Hq, Hkv, Dh = 4, 2, 64
    seqlens, kvlens = [5, 1, 9], [12, 30, 9]
    q, k, v, ss, ks = _case(rng, seqlens, kvlens, Hq, Hkv, Dh)
    mask = _mask_for(rng, sum(seqlens), sum(kvlens), Hq if per_head else None)
    mask[..., 3, 0:12] = -np.inf  # query row 3 (sequence 0) sees nothing
    for causal in (True, False):
        d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=3, is_causal=int(causal))
        got = orc.mha(d, q, k, v, ss, ks, attn_mask=mask).astype(np.float32)
        want = oracle_mod.np_mha(q, k, v, ss, ks, Hkv, causal, attn_mask=mask).astype(np.float32)
        assert np.isfinite(got).all() and not got[3].any()
        assert np.abs(got - want).max() <= 1e-3
        assert np.abs(got - orc.mha(d, q, k, v, ss, ks).astype(np.float32)).max() > 1e-2  # the mask does something


@pytest.mark.gpu
@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("causal", [True, False])
def test_gpu_attn_mask_matches_oracle(orc, dev, pkg, causal, per_head):
    import torch
    from ppl_nn_b200 import ops
    Hq, Hkv, Dh = 8, 2, 128
    seqlens, kvlens = [130, 7, 257, 1], [130, 40, 300, 77]
    rng = np.random.default_rng(23)
    q, k, v, ss, ks = _case(rng, seqlens, kvlens, Hq, Hkv, Dh)
    mask = _mask_for(rng, sum(seqlens), sum(kvlens), Hq if per_head else None)
    mask[..., 131, 130:170] = -np.inf  # a query row of sequence 1 that sees nothing
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=len(seqlens), is_causal=int(causal))
    want = orc.mha(d, q, k, v, ss, ks, attn_mask=mask).astype(np.float32)
    op = ops.MultiHeadAttention(ops.MultiHeadAttentionParam(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, is_causal=causal))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    got = op.forward(t(q), t(k), t(v), t(ss), t(ks), 0, max(seqlens), max(kvlens), attn_mask=t(mask))
    assert op.device_status() == 0
    got = got.cpu().numpy().astype(np.float32)
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max(), err.mean())


@pytest.mark.gpu
def test_gpu_host_operator_with_attn_mask(orc, dev, pkg, host):
    """The mask as input 8 of the host-layer operator (multi_head_attention_kernel.cc:30)."""
    import torch
    rng = np.random.default_rng(6)
    Hq, Hkv, Dh = 8, 2, 128
    q, k, v, ss, ks = _case(rng, [70, 3, 129], [70, 40, 129], Hq, Hkv, Dh)
    mask = _mask_for(rng, 202, 239)
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=3, is_causal=1)
    want = orc.mha(d, q, k, v, ss, ks, attn_mask=mask).astype(np.float32)
    eng = host.Engine(0, torch.cuda.current_stream().cuda_stream)
    op = host.Op(eng, "MultiHeadAttention", MHA_ATTRS)
    t = lambda a: torch.from_numpy(a).to(dev)
    out = torch.empty((q.shape[0], Hq, Dh), dtype=torch.float16, device=dev)
    op.run([t(q), t(k), t(v), t(ss), t(ks), 0, int(129), int(129), t(mask)], [out])
    eng.synchronize()
    err = np.abs(out.cpu().numpy().astype(np.float32) - want)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS
    op.close()
    eng.close()


@pytest.mark.gpu
def test_gpu_host_operator(orc, dev, pkg, host):
    import torch
    rng = np.random.default_rng(5)
    Hq, Hkv, Dh = 8, 2, 128
    q, k, v, ss, ks = _case(rng, [70, 3, 129], [70, 40, 129], Hq, Hkv, Dh)
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=3, is_causal=1)
    want = orc.mha(d, q, k, v, ss, ks).astype(np.float32)
    eng = host.Engine(0, torch.cuda.current_stream().cuda_stream)
    op = host.Op(eng, "MultiHeadAttention", MHA_ATTRS)
    t = lambda a: torch.from_numpy(a).to(dev)
    out = torch.empty((q.shape[0], Hq, Dh), dtype=torch.float16, device=dev)
    op.run([t(q), t(k), t(v), t(ss), t(ks), 0, int(129), int(129)], [out])
    eng.synchronize()
    err = np.abs(out.cpu().numpy().astype(np.float32) - want)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS
    op.close()
    eng.close()


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [True, False])
def test_gpu_agrees_with_torch_sdpa_fp32_at_size(dev, pkg, causal):
    """A second, independent reference at a size the CPU oracle does not reach in seconds: 3 sequences of
    up to 2 304 tokens, GQA 32/8 x 128, against torch's scaled_dot_product_attention in fp32 on the same GPU."""
    import torch
    from ppl_nn_b200 import ops
    Hq, Hkv, Dh = 32, 8, 128
    seqlens = [2304, 1000, 129]
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    T = sum(seqlens)
    q = torch.randn((T, Hq, Dh), generator=g, device=dev).to(torch.float16)
    k = torch.randn((T, Hkv, Dh), generator=g, device=dev).to(torch.float16)
    v = torch.randn((T, Hkv, Dh), generator=g, device=dev).to(torch.float16)
    ss = torch.tensor([0] + list(np.cumsum(seqlens)), dtype=torch.int64, device=dev)
    op = ops.MultiHeadAttention(ops.MultiHeadAttentionParam(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, is_causal=causal))
    got = op.forward(q, k, v, ss, ss.clone(), 0, max(seqlens), max(seqlens)).float()
    assert op.device_status() == 0
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for b, n in enumerate(seqlens):
            s0 = int(ss[b])
            qq = q[s0:s0 + n].float().transpose(0, 1)[None]
            kk = k[s0:s0 + n].float().repeat_interleave(Hq // Hkv, dim=1).transpose(0, 1)[None]
            vv = v[s0:s0 + n].float().repeat_interleave(Hq // Hkv, dim=1).transpose(0, 1)[None]
            with torch.nn.attention.sdpa_kernel(torch.nn.attention.SDPBackend.MATH):
                ref = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=causal)[0].transpose(0, 1)
            err = (got[s0:s0 + n] - ref).abs()
            assert float(err.max()) <= MAX_ABS and float(err.mean()) <= MEAN_ABS, (b, float(err.max()), float(err.mean()))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
