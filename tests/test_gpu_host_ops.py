"""GPU parity through the reference-facing operator interface: the C++ Op/Kernel classes created via
the registry (ppl.nn_b200/host), fed the 13-input / 10-input tensor lists of the reference's
operators, against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(built_lib, pkg):
    import torch
    from ppl_nn_b200 import hostapi
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    assert built_lib.device_ready()
    hostapi.register_ops()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    eng = hostapi.Engine(0, torch.cuda.current_stream().cuda_stream)
    yield hostapi, eng, dev
    eng.close()


def _device_array(ptr, shape, dev):
    """numpy copy of a kernel-allocated fp16 device buffer given by raw pointer."""
    import torch
    n = int(np.prod(shape))

    class _Raw:  # a torch-side view of the raw pointer
        __cuda_array_interface__ = {"shape": (n,), "typestr": "<f2", "data": (int(ptr), False), "version": 3}

    return torch.as_tensor(_Raw(), device=dev).clone().cpu().numpy().reshape(shape)


def _t(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


@pytest.mark.parametrize("layout,page,cache_prefill", [(0, 0, False), (3, 0, False), (0, 16, False), (0, 0, True)])
def test_mhca_and_kvcache_ops_match_the_oracle(orc, env, layout, page, cache_prefill):
    import torch
    from ppl_nn_b200 import workloads
    host, eng, dev = env
    assert eng.configure("cache_prefill", int(cache_prefill)) == "RC_SUCCESS"
    assert eng.configure("decoding_attn_split_k", 2) == "RC_SUCCESS"
    Hq, Hkv, Dh, L, l = 8, 2, 128, 2, 1
    idx = workloads.make_index([40, 300, 17, 1, 700], [100, 130], prefill_hist=[0, 64] if cache_prefill else None,
                               page_size=page)
    rng = np.random.default_rng(5)
    T = idx.total_tokens
    q = rng.standard_normal((T, Hq, Dh), dtype=np.float32).astype(np.float16)
    ck = rng.standard_normal((T, Hkv, Dh), dtype=np.float32).astype(np.float16)
    cv = rng.standard_normal((T, Hkv, Dh), dtype=np.float32).astype(np.float16)
    rows = int(idx.start_pos.sum())
    hk = rng.standard_normal((rows, Hkv, Dh), dtype=np.float32).astype(np.float16)
    hv = rng.standard_normal((rows, Hkv, Dh), dtype=np.float32).astype(np.float16)
    hstarts = np.concatenate([[0], np.cumsum(idx.start_pos)]).astype(np.int64)
    zeros = np.zeros_like(idx.start_pos)
    cshape, sshape = workloads.cache_shapes(layout, idx.max_tokens, L, Hkv, Dh)
    kw = dict(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, max_tokens=idx.max_tokens, num_layer=L,
              layer_idx=l, cache_layout=layout, cache_mode=1 if page else 0, page_size=page or 128,
              cachestart_stride_b=idx.cachestarts.shape[1] if page else 0, enable_cache_prefill=int(cache_prefill))
    # ---- oracle: history through KeyValueCache, then the attention op ----
    o_cache = np.zeros(cshape, dtype=np.int8)
    o_scale = np.zeros(sshape, dtype=np.float16)
    orc.kv_append(orc.desc(decoding_batches=0, **kw), hk, hv, hstarts, idx.cachestarts, zeros, o_cache, o_scale)
    want_key, want_value = orc.kv_gather_dequant(orc.desc(decoding_batches=0, **kw), hstarts, idx.cachestarts, o_cache,
                                                 o_scale)
    want = orc.mhca(orc.desc(decoding_batches=idx.decoding_batches, **kw), q, ck, cv, idx.seqstarts, idx.cachestarts,
                    idx.start_pos, o_cache, o_scale)
    # ---- host layer ----
    attrs = dict(num_layer=L, layer_idx=l, quant_bit=8, quant_group=8, cache_layout=layout, cache_mode=1 if page else 0,
                 page_size=page or 128)
    kvc = host.Op(eng, "KeyValueCache", attrs)
    mhca = host.Op(eng, "MultiHeadCacheAttention", dict(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, **attrs))
    cache = torch.zeros(cshape, dtype=torch.int8, device=dev)
    scale = torch.zeros(sshape, dtype=torch.float16, device=dev)
    cachestarts = _t(idx.cachestarts, dev)
    # KeyValueCache: 10 inputs, 2 outputs allocated by the kernel; shape inference reads kvstarts[-1]
    # back from the device
    res = kvc.run([_t(hk, dev), _t(hv, dev), _t(hstarts, dev), _t(hstarts, dev), cachestarts, _t(zeros, dev),
                   int(idx.start_pos.max()), int(idx.start_pos.max()), cache, scale], [None, None])
    eng.synchronize()
    assert [list(r.dims[:3]) for r in res] == [[rows, Hkv, Dh]] * 2 and all(r.data for r in res)
    for r, w in zip(res, (want_key, want_value)):
        got = _device_array(r.data, (rows, Hkv, Dh), dev)
        np.testing.assert_array_equal(got.view(np.uint16), w.view(np.uint16))
    # MultiHeadCacheAttention: 12 inputs (no attn_mask), decoding_batches/max_seqlen/max_kvlen as host scalars
    out = torch.zeros((T, Hq, Dh), dtype=torch.float16, device=dev)
    mhca.run([_t(q, dev), _t(ck, dev), _t(cv, dev), _t(idx.seqstarts, dev), _t(idx.kvstarts, dev), cachestarts,
              _t(idx.start_pos, dev), idx.decoding_batches, idx.max_seqlen, idx.max_kvlen, cache, scale], [out])
    eng.synchronize()
    np.testing.assert_array_equal(cache.cpu().numpy(), o_cache)
    np.testing.assert_array_equal(scale.cpu().numpy().view(np.uint16), o_scale.view(np.uint16))
    err = np.abs(out.cpu().numpy().astype(np.float32) - want.astype(np.float32))
    assert err.max() <= 2e-3 and err.mean() <= 1e-3, (err.max(), err.mean())
    assert eng.tmp_pool_bytes() > 0  # the workspace came from the engine's tmp-buffer pool
    kvc.close()
    mhca.close()


def test_host_scalars_on_the_device_are_read_with_a_sync(orc, env):
    """decoding_batches / max_seqlen / max_kvlen may live on the GPU; the kernel then copies them to the
    host (and synchronises) like the reference does."""
    import torch
    from ppl_nn_b200 import workloads
    host, eng, dev = env
    assert eng.configure("cache_prefill", 0) == "RC_SUCCESS"
    Hq, Hkv, Dh = 4, 4, 64
    idx = workloads.make_index([9, 33, 64], [])
    rng = np.random.default_rng(6)
    q = rng.standard_normal((3, Hq, Dh), dtype=np.float32).astype(np.float16)
    ck = rng.standard_normal((3, Hkv, Dh), dtype=np.float32).astype(np.float16)
    cv = rng.standard_normal((3, Hkv, Dh), dtype=np.float32).astype(np.float16)
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
    o_cache = rng.integers(-127, 128, size=cshape, dtype=np.int8)
    # |dequantised value| stays below 2, where one fp16 ulp of the output is still within the 2e-3 bound
    o_scale = rng.uniform(0.002, 0.012, size=sshape).astype(np.float16)
    cache, scale = _t(o_cache, dev), _t(o_scale, dev)
    want = orc.mhca(orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=3, decoding_batches=3,
                             max_tokens=idx.max_tokens), q, ck, cv, idx.seqstarts, idx.cachestarts, idx.start_pos,
                    o_cache, o_scale)
    op = host.Op(eng, "MultiHeadCacheAttention", dict(num_heads=Hq, head_dim=Dh, num_layer=1, layer_idx=0, quant_bit=8))
    out = torch.zeros((3, Hq, Dh), dtype=torch.float16, device=dev)
    scal = [torch.tensor(v, dtype=torch.int64, device=dev) for v in (3, 1, idx.max_kvlen)]
    op.run([_t(q, dev), _t(ck, dev), _t(cv, dev), _t(idx.seqstarts, dev), _t(idx.kvstarts, dev),
            _t(idx.cachestarts, dev), _t(idx.start_pos, dev), scal[0], scal[1], scal[2], cache, scale], [out])
    eng.synchronize()
    err = np.abs(out.cpu().numpy().astype(np.float32) - want.astype(np.float32))
    assert err.max() <= 2e-3 and err.mean() <= 1e-3
    op.close()


def test_attn_mask_is_input_12_of_the_host_operator(orc, env):
    """The optional mask travels through the host kernel as the reference forwards it
    (multi_head_cache_attention_kernel.cc:39,105-110): 13th input, fp16, [T, C]."""
    import torch
    from ppl_nn_b200 import workloads
    host, eng, dev = env
    assert eng.configure("cache_prefill", 0) == "RC_SUCCESS"
    Hq, Hkv, Dh = 8, 2, 128
    idx = workloads.make_index([9, 333, 64], [40])
    T, KV = idx.total_tokens, int(idx.kvstarts[-1])
    rng = np.random.default_rng(8)
    q = rng.standard_normal((T, Hq, Dh), dtype=np.float32).astype(np.float16)
    ck = rng.standard_normal((T, Hkv, Dh), dtype=np.float32).astype(np.float16)
    cv = rng.standard_normal((T, Hkv, Dh), dtype=np.float32).astype(np.float16)
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
    o_cache = rng.integers(-127, 128, size=cshape, dtype=np.int8)
    o_scale = rng.uniform(0.002, 0.012, size=sshape).astype(np.float16)
    cache, scale = _t(o_cache, dev), _t(o_scale, dev)
    mask = (rng.standard_normal((T, (KV + 7) // 8 * 8)) * 0.5).astype(np.float16)
    mask[rng.random(mask.shape) < 0.2] = -np.inf
    want = orc.mhca(orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, decoding_batches=3,
                             max_tokens=idx.max_tokens), q, ck, cv, idx.seqstarts, idx.cachestarts, idx.start_pos,
                    o_cache, o_scale, kvstarts=idx.kvstarts, attn_mask=mask)
    op = host.Op(eng, "MultiHeadCacheAttention", dict(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, num_layer=1,
                                                      layer_idx=0, quant_bit=8))
    out = torch.zeros((T, Hq, Dh), dtype=torch.float16, device=dev)
    op.run([_t(q, dev), _t(ck, dev), _t(cv, dev), _t(idx.seqstarts, dev), _t(idx.kvstarts, dev),
            _t(idx.cachestarts, dev), _t(idx.start_pos, dev), 3, idx.max_seqlen, idx.max_kvlen, cache, scale,
            _t(mask, dev)], [out])
    eng.synchronize()
    np.testing.assert_array_equal(cache.cpu().numpy(), o_cache)
    err = np.abs(out.cpu().numpy().astype(np.float32) - want.astype(np.float32))
    assert err.max() <= 2e-3 and err.mean() <= 1e-3, (err.max(), err.mean())
    op.close()
