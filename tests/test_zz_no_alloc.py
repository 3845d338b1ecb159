"""The workspace-free entry point, pplb200_mhca_forward_noalloc, against pplb200_mhca_forward.

Some users of this library cannot allocate device memory when they call the operator: an op that is
run outside its engine's device context has no tmp-buffer pool, and a serving process that has
handed all free memory to the KV cache (or that may not call cudaMalloc next to its own allocator)
has nothing to pass as `workspace`.  For them the library carries a fixed 32 MiB scratch array in
its device image.  This test calls the new entry point through the C ABI twice in a row, on two
different ragged batches that both need split partials in the scratch, and checks each output
against the ordinary entry point given a torch-allocated workspace.  It also checks that a call
whose scratch demand exceeds the array is refused with RC_OUT_OF_MEMORY.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-3
MEAN_ABS = 1e-3


def _device_inputs(dev, lens, prefill, hq, hkv, dh, seed):
    """A ragged batch on the device whose cache is written by the library's own append."""
    import torch
    from ppl_nn_b200 import workloads

    idx = workloads.make_index(lens, prefill)
    rng = np.random.default_rng(seed)
    T = idx.total_tokens

    def t(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    q = t(rng.standard_normal((T, hq, dh), dtype=np.float32).astype(np.float16))
    ck = t(rng.standard_normal((T, hkv, dh), dtype=np.float32).astype(np.float16))
    cv = t(rng.standard_normal((T, hkv, dh), dtype=np.float32).astype(np.float16))
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, hkv, dh)
    # any codes and scales are a valid cache; random ones are enough to compare two entry points
    cache = t(rng.integers(-127, 128, size=cshape, dtype=np.int8))
    scale = t(rng.uniform(0.005, 0.05, size=sshape).astype(np.float16))
    tensors = dict(q=q, ck=ck, cv=cv, seqstarts=t(idx.seqstarts), kvstarts=t(idx.kvstarts),
                   cachestarts=t(idx.cachestarts), start_pos=t(idx.start_pos), cache=cache, scale=scale)
    return idx, tensors


def _run_both(lib, op, dev, idx, x):
    import torch
    from ppl_nn_b200 import capi

    p = op.make_params(batch=idx.batch, decoding_batches=idx.decoding_batches, max_seqlen=idx.max_seqlen,
                       max_kvlen=idx.max_kvlen, total_tokens=idx.total_tokens, max_tokens=idx.max_tokens)
    rc, need = lib.mhca_workspace_size(p)
    assert rc == capi.SUCCESS
    assert 256 < need <= lib.static_scratch_bytes()
    stream = torch.cuda.current_stream().cuda_stream
    # the two entry points append into separate copies of the cache so that neither sees the other's work
    cache_a, scale_a = x["cache"].clone(), x["scale"].clone()
    cache_b, scale_b = x["cache"].clone(), x["scale"].clone()
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    ref = torch.zeros_like(x["q"])
    rc = lib.mhca_forward(p, x["q"].data_ptr(), x["ck"].data_ptr(), x["cv"].data_ptr(), x["seqstarts"].data_ptr(),
                          x["kvstarts"].data_ptr(), x["cachestarts"].data_ptr(), x["start_pos"].data_ptr(),
                          cache_a.data_ptr(), scale_a.data_ptr(), ws.data_ptr(), need, ref.data_ptr(), stream)
    assert rc == capi.SUCCESS
    got = torch.zeros_like(x["q"])
    rc = lib.mhca_forward_noalloc(p, x["q"].data_ptr(), x["ck"].data_ptr(), x["cv"].data_ptr(),
                                  x["seqstarts"].data_ptr(), x["kvstarts"].data_ptr(), x["cachestarts"].data_ptr(),
                                  x["start_pos"].data_ptr(), cache_b.data_ptr(), scale_b.data_ptr(), got.data_ptr(),
                                  stream)
    assert rc == capi.SUCCESS
    rc, status = lib.static_scratch_status(stream)  # the status word lives in the built-in scratch
    assert rc == capi.SUCCESS and status == 0
    torch.cuda.synchronize(dev)
    assert torch.equal(cache_a, cache_b) and torch.equal(scale_a, scale_b)
    r = ref.float().cpu().numpy()
    g = got.float().cpu().numpy()
    assert np.isfinite(g).all() and np.abs(r).max() > 0
    err = np.abs(g - r)
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max(), err.mean())


def test_noalloc_matches_workspace_entry_point_twice_in_a_row(built_lib, pkg):
    import torch
    from ppl_nn_b200 import ops

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    assert built_lib.device_ready()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    op = ops.MultiHeadCacheAttention(
        ops.MultiHeadCacheAttentionParam(num_heads=16, num_kv_heads=4, head_dim=128, num_layer=1, layer_idx=0,
                                         quant_bit=8),
        ops.EngineConfig(specify_decoding_attn_split_k=2))  # always split: the scratch holds partials
    # first call: long decode sequences (several splits each) plus two prefill sequences
    idx1, x1 = _device_inputs(dev, [3000, 517, 1, 2049, 4096, 1000], [70, 200], 16, 4, 128, seed=101)
    _run_both(built_lib, op, dev, idx1, x1)
    # second call, right after: a different batch, so stale partials from the first would show
    idx2, x2 = _device_inputs(dev, [129, 4000, 64, 3333], [], 16, 4, 128, seed=102)
    _run_both(built_lib, op, dev, idx2, x2)


def test_noalloc_rejects_calls_beyond_its_scratch(built_lib, pkg):
    import ctypes
    import torch
    from ppl_nn_b200 import ops

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    op = ops.MultiHeadCacheAttention(
        ops.MultiHeadCacheAttentionParam(num_heads=64, num_kv_heads=8, head_dim=128, num_layer=1, layer_idx=0,
                                         quant_bit=8),
        ops.EngineConfig(specify_decoding_attn_split_k=2, enable_cache_prefill=True))
    # 64 prefill sequences of up to 64k cached tokens each would need GBs of fp16 staging
    p = op.make_params(batch=4160, decoding_batches=4096, max_seqlen=4096, max_kvlen=65536, total_tokens=8192,
                       max_tokens=1 << 22)
    rc, need = built_lib.mhca_workspace_size(p)
    assert rc == 0 and need > built_lib.static_scratch_bytes()
    fake = ctypes.c_void_p(4096)  # never dereferenced: the size check comes first
    rc = built_lib.mhca_forward_noalloc(p, fake, fake, fake, fake, fake, fake, fake, fake, fake, fake, None)
    assert built_lib.status_str(rc) == "RC_OUT_OF_MEMORY"
