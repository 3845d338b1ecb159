"""The benchmark configurations at FULL size on the GPU, checked through properties that do not need
the CPU oracle to chew through gigabytes:
  * sampled sequences of the full ragged batch against the oracle on a compacted copy of their cache rows
    (cache codes/scales of the appended tokens bit-exact, attention within 2e-3 / 1e-3);
  * softmax weights sum to one: with every V row dequantising to the same vector, the output IS that
    vector, for every sequence and head of the batch;
  * split-k invariance: stream-k ranges, whole-segment scheduling and forced splitting agree;
  * linearity in V: doubling the V scales doubles the output bit for bit;
  * causality of the prefill: rewriting the tail of every prompt leaves the rows before it bit-identical;
  * append -> gather round trip within half a quantisation step for every new token."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-3
MEAN_ABS = 1e-3


@pytest.fixture(scope="module")
def dev(built_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    assert built_lib.device_ready()
    d = torch.device("cuda:0")
    torch.cuda.set_device(d)
    return d


def _op(dc, spec, split_k=1, cache_prefill=False):
    from ppl_nn_b200 import ops
    return ops.MultiHeadCacheAttention(
        ops.MultiHeadCacheAttentionParam(num_heads=dc.num_heads, num_kv_heads=dc.num_kv_heads, head_dim=spec.head_dim,
                                         num_layer=dc.num_layer, layer_idx=dc.layer_idx, quant_bit=8,
                                         cache_layout=dc.layout),
        ops.EngineConfig(specify_decoding_attn_split_k=split_k, enable_cache_prefill=cache_prefill))


def _forward(op, dc, **kw):
    idx = dc.index
    return op.forward(dc.query, dc.current_key, dc.current_value, dc.seqstarts, dc.kvstarts, dc.cachestarts,
                      dc.start_pos, idx.decoding_batches, idx.max_seqlen, idx.max_kvlen, dc.cache, dc.scale, **kw)


def _check_sample(orc, dc, spec, out, seqs, cache_prefill=False):
    """Oracle on the sequences `seqs` only, over a compacted host copy of their cache rows (layout 0)."""
    from ppl_nn_b200 import workloads
    idx = dc.index
    Hq, Hkv, Dh = dc.num_heads, dc.num_kv_heads, spec.head_dim
    kvl = idx.kvlens[seqs]
    n_dec = int(sum(1 for b in seqs if b < idx.decoding_batches))
    sub = workloads.make_index(kvl[:n_dec], idx.seqlens[seqs][n_dec:])
    cshape, sshape = workloads.cache_shapes(0, sub.max_tokens, 1, Hkv, Dh)
    cache = np.zeros(cshape, dtype=np.int8)
    scale = np.zeros(sshape, dtype=np.float16)
    gpu_cache_rows, gpu_scale_rows = [], []
    def rows(t, r0, n):
        """Rows r0 .. r0+n of the op's layer as (n, 1, 2, H, X), whatever the layout and layer count."""
        if dc.layout == 0:  # (MaxT, L, 2, H, X)
            return t[r0:r0 + n, dc.layer_idx][:, None].cpu().numpy()
        return t[dc.layer_idx, :, :, r0:r0 + n].permute(2, 0, 1, 3)[:, None].contiguous().cpu().numpy()  # (L, 2, H, MaxT, X)

    for i, b in enumerate(seqs):
        r0, n = int(idx.cachestarts[b]), int(kvl[i])
        c = rows(dc.cache, r0, n)
        s = rows(dc.scale, r0, n)
        cache[sub.cachestarts[i]:sub.cachestarts[i] + n] = c
        scale[sub.cachestarts[i]:sub.cachestarts[i] + n] = s
        gpu_cache_rows.append(c)
        gpu_scale_rows.append(s)
    tok = np.concatenate([np.arange(idx.seqstarts[b], idx.seqstarts[b + 1]) for b in seqs])
    q = dc.query[tok].cpu().numpy()
    ck = dc.current_key[tok].cpu().numpy()
    cv = dc.current_value[tok].cpu().numpy()
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=sub.batch, decoding_batches=n_dec,
                 max_tokens=sub.max_tokens, enable_cache_prefill=int(cache_prefill))
    want = orc.mhca(d, q, ck, cv, sub.seqstarts, sub.cachestarts, sub.start_pos, cache, scale)
    # the oracle re-appended this step's tokens into its copy: the GPU's rows must be identical
    for i, b in enumerate(seqs):
        n = int(kvl[i])
        np.testing.assert_array_equal(cache[sub.cachestarts[i]:sub.cachestarts[i] + n], gpu_cache_rows[i])
        np.testing.assert_array_equal(scale[sub.cachestarts[i]:sub.cachestarts[i] + n].view(np.uint16),
                                      gpu_scale_rows[i].view(np.uint16))
    got = out[tok].cpu().numpy().astype(np.float32)
    err = np.abs(got - want.astype(np.float32))
    # shown with `pytest -s`: the figures of the result table
    print(f"[parity] {spec.name}: {len(seqs)} sequences ({n_dec} decode), {tok.size} tokens: codes and scales "
          f"bit-exact, attention max-abs {err.max():.3e} mean-abs {err.mean():.3e}")
    assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS, (err.max(), err.mean(), seqs)


def _sample(idx, rng, k_dec, k_pre=0):
    nd = idx.decoding_batches
    order = np.argsort(idx.kvlens[:nd])
    picks = set(order[:2].tolist()) | set(order[-1:].tolist()) | set(rng.choice(nd, size=k_dec, replace=False).tolist())
    seqs = sorted(picks)
    if k_pre:
        pre = np.arange(nd, idx.batch)
        seqs += sorted(pre[np.argsort(idx.seqlens[nd:])[:k_pre]].tolist())
    return seqs


@pytest.mark.parametrize("name,k_dec,k_pre", [("cfg2_llama7b_decode", 5, 0), ("cfg3_llama8b_mixed", 4, 2),
                                              ("cfg4_llama70b_decode", 6, 0)])
def test_full_size_sampled_sequences_match_the_oracle(orc, dev, pkg, name, k_dec, k_pre):
    import torch
    from ppl_nn_b200 import workloads
    spec = workloads.SPECS[name]
    dc = workloads.device_case(spec, dev)
    op = _op(dc, spec)
    out = _forward(op, dc)
    assert op.device_status() == 0
    assert bool(torch.isfinite(out.float()).all())
    _check_sample(orc, dc, spec, out, _sample(dc.index, np.random.default_rng(7), k_dec, k_pre))
    # split-k invariance on the whole batch
    ref = out.float()
    for mode in (0, 2):
        other = _forward(_op(dc, spec, split_k=mode), dc).float()
        diff = (other - ref).abs()
        assert float(diff.max()) <= MAX_ABS and float(diff.mean()) <= MEAN_ABS, (name, mode)
    del dc, out
    torch.cuda.empty_cache()


def test_cache_prefill_at_full_size(orc, dev, pkg):
    """The mixed continuous-batching step with enable_cache_prefill: the 8 prompts (512..2048 tokens) read their
    keys and values back from the INT8 cache.  The two shortest prompts and sampled decode sequences against the
    oracle; every prompt's output must also stay within tolerance of the run that reads the fp16 inputs, from
    which it differs only by the quantisation of K and V."""
    import torch
    from ppl_nn_b200 import workloads
    spec = workloads.SPECS["cfg3_llama8b_mixed"]
    dc = workloads.device_case(spec, dev)
    idx = dc.index
    op = _op(dc, spec, cache_prefill=True)
    out = _forward(op, dc)
    assert op.device_status() == 0
    assert bool(torch.isfinite(out.float()).all())
    _check_sample(orc, dc, spec, out, _sample(idx, np.random.default_rng(8), 2, 2), cache_prefill=True)
    plain = _forward(_op(dc, spec), dc).float()
    t0 = int(idx.seqstarts[idx.decoding_batches])
    diff = (out.float()[t0:] - plain[t0:]).abs()
    assert 0.0 < float(diff.max()) <= 0.25 and float(diff.mean()) <= 5e-3  # int8 K/V against fp16 K/V
    assert bool((out[:t0].view(torch.int16) == plain.to(torch.float16)[:t0].view(torch.int16)).all())  # decode rows: same
    del dc, out, plain
    torch.cuda.empty_cache()


@pytest.mark.parametrize("layout", [0, 3])
def test_cache_offsets_beyond_4_gib(orc, dev, pkg, layout):
    """The last layer of a 32-layer cache of 80 k token rows: 5.2 GB of codes, so the rows of that layer lie
    beyond 2^32 bytes in either layout (layout 0: row stride 64 KiB; layout 3: layer stride 164 MB).  Sampled
    sequences against the oracle, and no other layer of the cache may have been written."""
    import torch
    from ppl_nn_b200 import workloads
    spec = workloads.Spec("wide_cache", 32, 8, 128, 48, 1024, 2304, seed=9)
    L = 32
    dc = workloads.device_case(spec, dev, layout=layout, num_layer=L, layer_idx=L - 1)
    assert dc.cache.numel() > (1 << 32)
    op = _op(dc, spec)
    out = _forward(op, dc)
    assert op.device_status() == 0
    _check_sample(orc, dc, spec, out, _sample(dc.index, np.random.default_rng(3), 3))
    other = dc.cache[:, :L - 1] if layout == 0 else dc.cache[:L - 1]
    assert not bool(other.any())
    del dc, out, other
    torch.cuda.empty_cache()


def test_long_context_full_size(orc, dev, pkg):
    """16 sequences of 32k..128k cached tokens with peaked softmax: the shortest and the LONGEST one (where
    split-k merges the most partials) against the oracle, all of them for split-k invariance, and the appended
    token of every sequence bit-exact."""
    import torch
    from ppl_nn_b200 import workloads
    spec = workloads.SPECS["cfg5_longctx"]
    dc = workloads.device_case(spec, dev)
    op = _op(dc, spec)
    out = _forward(op, dc)
    assert op.device_status() == 0
    shortest, longest = int(np.argmin(dc.index.kvlens)), int(np.argmax(dc.index.kvlens))
    _check_sample(orc, dc, spec, out, [shortest, longest])
    other = _forward(_op(dc, spec, split_k=0), dc).float()
    diff = (other - out.float()).abs()
    assert float(diff.max()) <= MAX_ABS and float(diff.mean()) <= MEAN_ABS
    del dc, out
    torch.cuda.empty_cache()


def test_softmax_weights_sum_to_one_at_full_size(dev, pkg):
    """All V rows of the cache dequantise to the same vector v (per head); whatever the scores are, the
    output must be v for every sequence and head: 256 sequences x 32 heads of the LLaMA-2-7B workload."""
    import torch
    from ppl_nn_b200 import capi, workloads
    spec = workloads.SPECS["cfg2_llama7b_decode"]
    dc = workloads.device_case(spec, dev)
    Hkv, Dh = dc.num_kv_heads, spec.head_dim
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    codes = torch.randint(-127, 128, (Hkv, Dh), generator=g, device=dev, dtype=torch.int8)
    scales = (torch.rand((Hkv, Dh // 8), generator=g, device=dev) * 0.01 + 0.002).to(torch.float16)
    dc.cache[:, 0, 1] = codes   # (MaxT, L, 2, H, Dh): every V row
    dc.scale[:, 0, 1] = scales
    v = (codes.float().view(Hkv, Dh // 8, 8) * scales.float()[..., None]).view(Hkv, Dh)
    # the step's own V token would overwrite one row per sequence: skip the append, attend to the cache as it is
    op = _op(dc, spec)
    out = _forward(op, dc, phase_mask=capi.PHASE_DECODE)
    assert op.device_status() == 0
    want = v.to(torch.float16).float()[None].expand(out.shape[0], -1, -1)
    diff = (out.float() - want).abs()
    # one fp16 ulp of |v| < 2 at most: the fp32 sum of p*v over p-sum may round the other way
    assert float(diff.max()) <= 2.0 ** -10 + 1e-7, float(diff.max())
    assert float((diff > 0).float().mean()) < 0.05
    del dc, out
    torch.cuda.empty_cache()


def test_output_is_linear_in_v_at_full_size(dev, pkg):
    """Doubling every V scale of the cache (a power of two, so every product and every partial sum doubles
    exactly) must double the output bit for bit: 512 sequences x 64 heads of the LLaMA-2-70B workload, whatever
    the split points and partial merges are."""
    import torch
    from ppl_nn_b200 import capi, workloads
    spec = workloads.SPECS["cfg4_llama70b_decode"]
    dc = workloads.device_case(spec, dev)
    op = _op(dc, spec)
    once = _forward(op, dc, phase_mask=capi.PHASE_DECODE).clone()   # attend to the cache as it is, no append
    dc.scale[:, 0, 1] *= 2                                          # (MaxT, L, 2, H, Dh/8): the V scales
    twice = _forward(op, dc, phase_mask=capi.PHASE_DECODE)
    assert op.device_status() == 0
    a, b = once.float(), twice.float()
    normal = a.abs() >= 2.0 ** -13                                  # 2x of a subnormal half need not be exact
    assert bool(normal.float().mean() > 0.9)
    assert bool((b[normal] == 2 * a[normal]).all())
    del dc, once, twice
    torch.cuda.empty_cache()


def test_prefill_is_causal_at_full_size(dev, pkg):
    """The 8 prompts of the mixed configuration (512 .. 2048 tokens): overwriting the last 100 tokens of every
    prompt (query, key and value) must leave the output rows before them bit-identical, whichever CTA computed
    them and in whatever order the tiles were drawn."""
    import torch
    from ppl_nn_b200 import workloads
    spec = workloads.SPECS["cfg3_prefill_only"]
    dc = workloads.device_case(spec, dev)
    idx = dc.index
    op = _op(dc, spec)
    before = _forward(op, dc).clone()
    assert op.device_status() == 0
    keep = torch.ones(dc.query.shape[0], dtype=torch.bool, device=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    for b in range(idx.batch):
        lo, hi = int(idx.seqstarts[b + 1]) - 100, int(idx.seqstarts[b + 1])
        keep[lo:hi] = False
        for t in (dc.query, dc.current_key, dc.current_value):
            t[lo:hi] = torch.randn(t[lo:hi].shape, generator=g, device=dev).to(torch.float16)
    after = _forward(op, dc)
    assert op.device_status() == 0
    assert bool((before[keep].view(torch.int16) == after[keep].view(torch.int16)).all())
    assert not bool((before[~keep].view(torch.int16) == after[~keep].view(torch.int16)).all())
    del dc, before, after
    torch.cuda.empty_cache()


def test_append_gather_round_trip_at_full_size(dev, pkg):
    """KeyValueCache on the 512-sequence LLaMA-2-70B workload: the dequantised history returned by the
    op holds, in the last row of every sequence, this step's token within half a quantisation step."""
    import torch
    from ppl_nn_b200 import ops, workloads
    spec = workloads.SPECS["cfg4_llama70b_decode"]
    dc = workloads.device_case(spec, dev)
    idx = dc.index
    kvc = ops.KeyValueCache(ops.KeyValueCacheParam(num_layer=1, layer_idx=0, quant_bit=8))
    key, value = kvc.forward(dc.current_key, dc.current_value, dc.seqstarts, dc.kvstarts, dc.cachestarts, dc.start_pos,
                             idx.max_seqlen, idx.max_kvlen, dc.cache, dc.scale)
    assert key.shape == (int(idx.kvstarts[-1]), dc.num_kv_heads, spec.head_dim)
    last = torch.from_numpy(idx.kvstarts[1:] - 1).to(dev)
    for full, cur in ((key, dc.current_key), (value, dc.current_value)):
        got = full.index_select(0, last).float()
        x = cur.float()
        step = x.view(x.shape[0], x.shape[1], -1, 8).abs().amax(-1, keepdim=True) / 127.0
        bound = (0.5 * step * (1 + 2.0 ** -9) + x.view_as(step.expand(-1, -1, -1, 8)).abs() * 2.0 ** -10 + 1e-6)
        err = (got - x).view_as(bound).abs()
        assert bool((err <= bound).all())
    del dc, key, value
    torch.cuda.empty_cache()
