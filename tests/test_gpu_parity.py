"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded
inputs.  Cache codes and scales must be bit-exact; attention must be within 2e-3 max-abs and 1e-3
mean-abs (the tolerance the task states for this floating-point kernel)."""
from dataclasses import replace

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-3
MEAN_ABS = 1e-3


@pytest.fixture(scope="module")
def torch_dev(built_lib):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    assert built_lib.device_ready(), "the CUDA library has no sm_100a code for this device"
    return torch.device("cuda:0")


def _t(a, dev):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def run_case(orc, dev, hc, *, layout=0, num_layer=1, layer_idx=0, split_k=1, cache_prefill=False,
             check_attention=True, attn_mask=None):
    """History append + one MultiHeadCacheAttention call on both sides; returns the error stats."""
    import torch
    from ppl_nn_b200 import ops, workloads

    idx, hidx = hc.index, hc.hist_index
    Hq, Hkv, Dh = hc.num_heads, hc.num_kv_heads, hc.spec.head_dim
    page = idx.page_size
    cshape, sshape = workloads.cache_shapes(layout, idx.max_tokens, num_layer, Hkv, Dh)
    kw = dict(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, max_tokens=idx.max_tokens,
              num_layer=num_layer, layer_idx=layer_idx, cache_layout=layout, cache_mode=1 if page else 0,
              page_size=page or 128, cachestart_stride_b=idx.cachestarts.shape[1] if page else 0,
              is_causal=int(hc.spec.is_causal), enable_cache_prefill=int(cache_prefill))
    # ---- oracle ----
    o_cache = np.zeros(cshape, dtype=np.int8)
    o_scale = np.zeros(sshape, dtype=np.float16)
    orc.kv_append(orc.desc(decoding_batches=0, **kw), hc.hist_key, hc.hist_value, hidx.seqstarts, hidx.cachestarts,
                  hidx.start_pos, o_cache, o_scale)
    want = orc.mhca(orc.desc(decoding_batches=idx.decoding_batches, **kw), hc.query, hc.current_key,
                    hc.current_value, idx.seqstarts, idx.cachestarts, idx.start_pos, o_cache, o_scale,
                    kvstarts=idx.kvstarts, attn_mask=attn_mask)
    # ---- CUDA ----
    cache = torch.zeros(cshape, dtype=torch.int8, device=dev)
    scale = torch.zeros(sshape, dtype=torch.float16, device=dev)
    kvc = ops.KeyValueCache(ops.KeyValueCacheParam(num_layer=num_layer, layer_idx=layer_idx, quant_bit=8,
                                                   cache_layout=layout, cache_mode=1 if page else 0,
                                                   page_size=page or 128))
    if hidx.total_tokens > 0:
        kvc.forward(_t(hc.hist_key, dev), _t(hc.hist_value, dev), _t(hidx.seqstarts, dev), _t(hidx.kvstarts, dev),
                    _t(hidx.cachestarts, dev), _t(hidx.start_pos, dev), hidx.max_seqlen, hidx.max_kvlen, cache, scale,
                    total_kv=0)
    op = ops.MultiHeadCacheAttention(
        ops.MultiHeadCacheAttentionParam(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, num_layer=num_layer,
                                         layer_idx=layer_idx, quant_bit=8, cache_layout=layout,
                                         cache_mode=1 if page else 0, page_size=page or 128,
                                         is_causal=hc.spec.is_causal),
        ops.EngineConfig(enable_cache_prefill=cache_prefill, specify_decoding_attn_split_k=split_k))
    got = op.forward(_t(hc.query, dev), _t(hc.current_key, dev), _t(hc.current_value, dev), _t(idx.seqstarts, dev),
                     _t(idx.kvstarts, dev), _t(idx.cachestarts, dev), _t(idx.start_pos, dev), idx.decoding_batches,
                     idx.max_seqlen, idx.max_kvlen, cache, scale,
                     attn_mask=None if attn_mask is None else _t(attn_mask, dev))
    assert op.device_status() == 0
    np.testing.assert_array_equal(cache.cpu().numpy(), o_cache, err_msg="INT8 cache codes differ")
    np.testing.assert_array_equal(scale.cpu().numpy().view(np.uint16), o_scale.view(np.uint16),
                                  err_msg="fp16 cache scales differ")
    got = got.cpu().numpy().astype(np.float32)
    run_case.last_output = got
    assert np.isfinite(got).all()
    err = np.abs(got - want.astype(np.float32))
    if check_attention:
        per_seq = [float(err[idx.seqstarts[b]:idx.seqstarts[b + 1]].max()) if idx.seqstarts[b + 1] > idx.seqstarts[b]
                   else 0.0 for b in range(idx.batch)]
        worst = int(np.argmax(per_seq))
        assert err.max() <= MAX_ABS, (f"max-abs {err.max():.3e}; worst sequence {worst} kvlen "
                                      f"{int(idx.kvlens[worst])} seqlen {int(idx.seqlens[worst])}")
        assert err.mean() <= MEAN_ABS
    return err, op


def _spec(**kw):
    from ppl_nn_b200 import workloads
    base = workloads.Spec("custom", 8, 8, 128, 4, 1, 64)
    return replace(base, **kw)


def test_cfg1_tiny_decode(orc, torch_dev, pkg):
    from ppl_nn_b200 import workloads
    hc = workloads.host_case(workloads.SPECS["cfg1_tiny"])
    err, _ = run_case(orc, torch_dev, hc)
    # and against the committed golden output of the oracle
    from pathlib import Path
    g = Path(__file__).resolve().parent / "golden" / "attn_output-4_8_64-fp16.dat"
    want = np.fromfile(g, dtype=np.float16).reshape(4, 8, 64).astype(np.float32)
    got = run_case.last_output
    assert got.shape == want.shape
    gerr = np.abs(got - want)
    assert gerr.max() <= MAX_ABS and gerr.mean() <= MEAN_ABS, (gerr.max(), gerr.mean())


@pytest.mark.parametrize("layout,num_layer,layer_idx", [(0, 1, 0), (3, 1, 0), (0, 3, 1), (3, 2, 1)])
def test_cfg2_mha_outlier_channels(orc, torch_dev, pkg, layout, num_layer, layer_idx):
    from ppl_nn_b200 import workloads
    spec = workloads.scaled(workloads.SPECS["cfg2_llama7b_decode"], seqs=24 / 256, length=0.25)
    run_case(orc, torch_dev, workloads.host_case(spec), layout=layout, num_layer=num_layer, layer_idx=layer_idx)


@pytest.mark.parametrize("dh", [128, 64])
def test_one_head_per_kv_head_both_score_paths(orc, torch_dev, pkg, dh, monkeypatch):
    """With one query head per kv head the decode kernel takes the scores from integer dot products
    (codes x int16-quantised query) instead of the tensor cores; PPLB200_DECODE_KDOT=0 (read per call) sends
    the same batch through the tensor-core scores.  Both must meet the tolerance, and they must agree with
    one another far more closely than that (they differ only in how the keys are weighted, not in V)."""
    from ppl_nn_b200 import workloads
    spec = replace(workloads.scaled(workloads.SPECS["cfg2_llama7b_decode"], seqs=16 / 256, length=0.2), num_heads=8,
                   num_kv_heads=8, head_dim=dh)
    hc = workloads.host_case(spec)
    outs = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("PPLB200_DECODE_KDOT", flag)
        run_case(orc, torch_dev, hc)
        outs[flag] = run_case.last_output.copy()
    assert np.abs(outs["1"] - outs["0"]).max() <= MAX_ABS


@pytest.mark.parametrize("world", [1, 2, 8])
def test_cfg4_gqa8_kv_head_shards(orc, torch_dev, pkg, world):
    """64 query / 8 kv heads, sharded by kv head: 8, 4 and 1 kv heads per rank exercise all three
    warp arrangements of the decode kernel."""
    from ppl_nn_b200 import workloads
    spec = workloads.scaled(workloads.SPECS["cfg4_llama70b_decode"], seqs=32 / 512, length=0.25)
    for rank in sorted({0, world - 1}):
        run_case(orc, torch_dev, workloads.host_case(spec, rank=rank, world=world))


@pytest.mark.parametrize("split_k", [0, 1, 2])
def test_cfg5_long_context_split_k(orc, torch_dev, pkg, split_k):
    from ppl_nn_b200 import workloads
    spec = workloads.scaled(workloads.SPECS["cfg5_longctx"], seqs=6 / 16, length=1 / 16)
    run_case(orc, torch_dev, workloads.host_case(spec), split_k=split_k)


@pytest.mark.parametrize("hq,hkv,dh", [(8, 8, 128), (8, 2, 128), (4, 4, 64), (16, 1, 128), (6, 2, 64)])
@pytest.mark.parametrize("split_k", [1, 2])
def test_every_length_1_to_80(orc, torch_dev, pkg, hq, hkv, dh, split_k):
    """Every kv length from 1 to 80 in one batch: every fill level of the 16-token tile, the 64-token
    chunk boundary and one above/below it, for MHA, GQA 4, GQA 16 (two head octets) and GQA 3."""
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=hq, num_kv_heads=hkv, head_dim=dh, n_decode=80, kv_dist="list",
                 kv_list=tuple(range(1, 81)), seed=21)
    run_case(orc, torch_dev, workloads.host_case(spec), split_k=split_k)


def test_split_boundaries(orc, torch_dev, pkg):
    """Lengths on, one below and one above the split size that the heuristic picks."""
    from ppl_nn_b200 import workloads
    lens = (191, 192, 193, 300, 1, 255, 256, 257, 383, 384, 385)
    spec = _spec(num_heads=8, num_kv_heads=2, head_dim=128, n_decode=len(lens), kv_dist="list", kv_list=lens, seed=22)
    for split_k in (0, 2):
        run_case(orc, torch_dev, workloads.host_case(spec), split_k=split_k)


@pytest.mark.parametrize("hq,hkv", [(8, 4), (4, 4)])  # tensor-core scores, and integer-dot scores (one head per kv head)
@pytest.mark.parametrize("page,layout", [(16, 0), (128, 0), (32, 3), (48, 0)])
def test_paged_cache(orc, torch_dev, pkg, page, layout, hq, hkv):
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=hq, num_kv_heads=hkv, head_dim=128, n_decode=12, kv_lo=1, kv_hi=700, seed=23)
    run_case(orc, torch_dev, workloads.host_case(spec, page_size=page), layout=layout, split_k=2)


def test_append_adversarial_values_bit_exact(orc, torch_dev, pkg):
    """+-65504, subnormals, zeros, -0.0, one outlier, all-equal, NaN and Inf groups."""
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=4, num_kv_heads=4, head_dim=64, n_decode=6, kv_dist="list", kv_list=(3, 9, 17, 33, 5, 64),
                 seed=24)
    hc = workloads.host_case(spec)
    rng = np.random.default_rng(5)
    for arr in (hc.hist_key, hc.hist_value, hc.current_key, hc.current_value):
        flat = arr.reshape(-1, 8)
        n = flat.shape[0]
        flat[rng.integers(0, n, 40), rng.integers(0, 8, 40)] = np.float16(65504)
        flat[rng.integers(0, n, 40), rng.integers(0, 8, 40)] = np.float16(-65504)
        flat[rng.integers(0, n, 40)] = np.float16(6e-8)
        flat[rng.integers(0, n, 40)] = np.float16(0)
        flat[rng.integers(0, n, 40)] = np.float16(-0.0)
        flat[rng.integers(0, n, 40)] = np.float16(0.37)
        flat[rng.integers(0, n, 40), rng.integers(0, 8, 40)] *= np.float16(300)
        flat[rng.integers(0, n, 10), rng.integers(0, 8, 10)] = np.float16("nan")
        flat[rng.integers(0, n, 10), rng.integers(0, 8, 10)] = np.float16("inf")
    import torch
    from ppl_nn_b200 import ops
    idx, hidx = hc.index, hc.hist_index
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, 4, 64)
    o_cache = np.zeros(cshape, dtype=np.int8)
    o_scale = np.zeros(sshape, dtype=np.float16)
    kw = dict(num_heads=4, num_kv_heads=4, head_dim=64, batch=idx.batch, max_tokens=idx.max_tokens)
    orc.kv_append(orc.desc(decoding_batches=0, **kw), hc.hist_key, hc.hist_value, hidx.seqstarts, hidx.cachestarts,
                  hidx.start_pos, o_cache, o_scale)
    orc.kv_append(orc.desc(decoding_batches=idx.batch, **kw), hc.current_key, hc.current_value, idx.seqstarts,
                  idx.cachestarts, idx.start_pos, o_cache, o_scale)
    dev = torch_dev
    cache = torch.zeros(cshape, dtype=torch.int8, device=dev)
    scale = torch.zeros(sshape, dtype=torch.float16, device=dev)
    kvc = ops.KeyValueCache(ops.KeyValueCacheParam(num_layer=1, layer_idx=0, quant_bit=8))
    kvc.forward(_t(hc.hist_key, dev), _t(hc.hist_value, dev), _t(hidx.seqstarts, dev), _t(hidx.kvstarts, dev),
                _t(hidx.cachestarts, dev), _t(hidx.start_pos, dev), hidx.max_seqlen, hidx.max_kvlen, cache, scale,
                total_kv=0)
    key, value = kvc.forward(_t(hc.current_key, dev), _t(hc.current_value, dev), _t(idx.seqstarts, dev),
                             _t(idx.kvstarts, dev), _t(idx.cachestarts, dev), _t(idx.start_pos, dev), idx.max_seqlen,
                             idx.max_kvlen, cache, scale)
    np.testing.assert_array_equal(cache.cpu().numpy(), o_cache)
    np.testing.assert_array_equal(scale.cpu().numpy().view(np.uint16), o_scale.view(np.uint16))
    # the operator's key/value outputs: dequantised history, bit-exact (NaN patterns aside)
    wk, wv = orc.kv_gather_dequant(orc.desc(decoding_batches=idx.batch, **kw), idx.kvstarts, idx.cachestarts, o_cache,
                                   o_scale)
    for got, want in ((key, wk), (value, wv)):
        g = got.cpu().numpy()
        assert g.shape == want.shape
        nan = np.isnan(want)
        np.testing.assert_array_equal(np.isnan(g), nan)
        np.testing.assert_array_equal(g[~nan].view(np.uint16), want[~nan].view(np.uint16))


def test_workspace_too_small_and_bad_params_are_rejected(torch_dev, built_lib, pkg):
    import torch
    from ppl_nn_b200 import capi, ops
    op = ops.MultiHeadCacheAttention(ops.MultiHeadCacheAttentionParam(num_heads=8, num_kv_heads=8, head_dim=128,
                                                                     num_layer=1, layer_idx=0, quant_bit=8))
    p = op.make_params(batch=4, decoding_batches=4, max_seqlen=1, max_kvlen=100000, total_tokens=4, max_tokens=1 << 20)
    rc, need = built_lib.mhca_workspace_size(p)
    assert rc == capi.SUCCESS and need > 256
    buf = torch.zeros(512, dtype=torch.uint8, device=torch_dev)
    one = torch.zeros(64, dtype=torch.int64, device=torch_dev)
    rc = built_lib.mhca_forward(p, one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(), buf.data_ptr(), 256,
                                one.data_ptr(), 0)
    assert built_lib.status_str(rc) == "RC_OUT_OF_MEMORY"
    rc = built_lib.mhca_forward(p, one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                one.data_ptr(), one.data_ptr(), one.data_ptr(), None, buf.data_ptr(), need,
                                one.data_ptr(), 0)
    assert built_lib.status_str(rc) == "RC_UNSUPPORTED"  # scale missing


@pytest.mark.parametrize("hq,hkv", [(8, 2), (4, 4), (12, 4), (16, 16)])
@pytest.mark.parametrize("layout,num_layer,layer_idx", [(3, 1, 0), (0, 2, 1)])
@pytest.mark.parametrize("split_k", [0, 1, 2])
def test_strided_cache_rows_with_2_4_and_8_head_lanes(orc, torch_dev, pkg, hq, hkv, layout, num_layer, layer_idx, split_k):
    """Caches whose token rows are strided (layout 3, or more than one layer) make the decode warps that
    share a range meet at a barrier after every tile.  With 2 or 4 kv heads a CTA holds several such
    groups, each on its own range, of different lengths when split-k is off."""
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=hq, num_kv_heads=hkv, head_dim=128, n_decode=80, kv_dist="list",
                 kv_list=tuple(range(1, 400, 5)), seed=23)
    run_case(orc, torch_dev, workloads.host_case(spec), layout=layout, num_layer=num_layer, layer_idx=layer_idx,
             split_k=split_k)


# ------------------------------------------------------------------------------------------------
# prefill (tcgen05) and mixed batches
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("hq,hkv,dh,lens", [
    (4, 4, 128, (128,)),                       # exactly one tile
    (4, 2, 128, (1, 5, 127, 129, 200)),        # ragged tails around the 128-row tile
    (8, 2, 64, (33, 256, 300)),                # head_dim 64
    (32, 8, 128, (515, 700)),                  # the LLaMA-3-8B head geometry, several kv tiles
])
def test_prefill_only(orc, torch_dev, pkg, hq, hkv, dh, lens):
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=hq, num_kv_heads=hkv, head_dim=dh, n_decode=0, kv_dist="list", kv_list=(),
                 n_prefill=len(lens), seed=31)
    hc = workloads.host_case(spec)
    # draw_lengths gives random prefill lengths; rebuild the case with the lengths we want
    idx = workloads.make_index([], lens)
    hc = _case_with_index(hc, idx, spec)
    run_case(orc, torch_dev, hc)


def test_prefill_many_short_sequences_through_the_tile_ring(orc, torch_dev, pkg):
    """400 prompts of 1..290 tokens: 4 800 tile indices for 296 persistent CTAs, two thirds of them beyond
    the end of their sequence (dropped by the producer warp), so every CTA draws many tiles, wraps the
    tile ring several times and changes between 1-, 2- and 5-block tiles."""
    from ppl_nn_b200 import workloads
    lens = tuple(1 + (37 * i) % 290 for i in range(400))
    spec = _spec(num_heads=4, num_kv_heads=2, head_dim=128, n_decode=0, kv_dist="list", kv_list=(),
                 n_prefill=len(lens), seed=33)
    hc = workloads.host_case(spec)
    hc = _case_with_index(hc, workloads.make_index([], lens), spec)
    run_case(orc, torch_dev, hc)


def _case_with_index(hc, idx, spec, prefill_hist=None):
    """Re-draw the tensors of a HostCase for an explicit index."""
    from ppl_nn_b200 import workloads
    rng = np.random.default_rng([spec.seed, 77])
    T = idx.total_tokens
    hk, hq, dh = hc.num_kv_heads, hc.num_heads, spec.head_dim
    hc.index = idx
    hc.query = rng.standard_normal((T, hq, dh), dtype=np.float32).astype(np.float16)
    hc.current_key = rng.standard_normal((T, hk, dh), dtype=np.float32).astype(np.float16)
    hc.current_value = rng.standard_normal((T, hk, dh), dtype=np.float32).astype(np.float16)
    rows = int(idx.start_pos.sum())
    hc.hist_key = rng.standard_normal((rows, hk, dh), dtype=np.float32).astype(np.float16)
    hc.hist_value = rng.standard_normal((rows, hk, dh), dtype=np.float32).astype(np.float16)
    starts = np.concatenate([[0], np.cumsum(idx.start_pos)]).astype(np.int64)
    hc.hist_index = workloads.Index(seqstarts=starts, kvstarts=starts.copy(), cachestarts=idx.cachestarts,
                                    start_pos=np.zeros_like(idx.start_pos), seqlens=idx.start_pos.copy(),
                                    decoding_batches=0, max_seqlen=int(idx.start_pos.max()) if idx.batch else 0,
                                    max_kvlen=int(idx.start_pos.max()) if idx.batch else 0, total_tokens=rows,
                                    max_tokens=idx.max_tokens, page_size=idx.page_size)
    return hc


def test_cfg3_mixed_decode_and_prefill(orc, torch_dev, pkg):
    """248 decode + 8 prefill sequences in one ragged call, scaled down: GQA 32/8, causal."""
    from ppl_nn_b200 import workloads
    spec = workloads.scaled(workloads.SPECS["cfg3_llama8b_mixed"], seqs=24 / 256, length=0.125)
    hc = workloads.host_case(spec)
    assert hc.index.decoding_batches > 0 and hc.index.batch > hc.index.decoding_batches
    run_case(orc, torch_dev, hc)


@pytest.mark.parametrize("layout", [0, 3])
def test_cache_prefill_with_history(orc, torch_dev, pkg, layout):
    """enable_cache_prefill: prefill sequences with start_pos > 0 read the INT8 cache (chunked
    prefill), next to decode sequences in the same call."""
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=8, num_kv_heads=2, head_dim=128, n_decode=3, kv_dist="list", kv_list=(40, 300, 17),
                 n_prefill=3, seed=33)
    hc = workloads.host_case(spec)
    idx = workloads.make_index([40, 300, 17], [100, 64, 130], prefill_hist=[0, 200, 131])
    hc = _case_with_index(hc, idx, spec)
    run_case(orc, torch_dev, hc, layout=layout, cache_prefill=True)


@pytest.mark.parametrize("cache_prefill", [False, True])
def test_non_causal_prefill_in_the_cached_operator(orc, torch_dev, pkg, cache_prefill):
    """is_causal = 0 is passed through (multi_head_cache_attention_kernel.cc:184 passes param_->is_causal):
    every query row of a prefill sequence sees all of the sequence's kv positions; decode rows are unaffected."""
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=8, num_kv_heads=2, head_dim=128, n_decode=2, kv_dist="list", kv_list=(40, 300),
                 n_prefill=3, seed=34, is_causal=False)
    hc = workloads.host_case(spec)
    idx = workloads.make_index([40, 300], [100, 64, 200], prefill_hist=[0, 77, 0] if cache_prefill else None)
    hc = _case_with_index(hc, idx, spec)
    run_case(orc, torch_dev, hc, cache_prefill=cache_prefill)


def _random_mask(rng, idx, heads=None, cols_extra=0):
    """Additive fp16 mask [T, C] (or [heads, T, C]): small biases, about a fifth of the entries -inf, one query
    row with every position removed, columns padded up to a multiple of 8 (plus `cols_extra`)."""
    T, KV = idx.total_tokens, int(idx.kvstarts[-1])
    C = (KV + 7) // 8 * 8 + cols_extra
    shape = (T, C) if heads is None else (heads, T, C)
    m = (rng.standard_normal(shape) * 0.5).astype(np.float16)
    m[rng.random(shape) < 0.2] = -np.inf
    b = idx.batch - 1  # the first query row of the last sequence sees nothing at all
    m[..., int(idx.seqstarts[b]), int(idx.kvstarts[b]):int(idx.kvstarts[b + 1])] = -np.inf
    return m


@pytest.mark.parametrize("per_head", [False, True])
@pytest.mark.parametrize("cache_prefill", [False, True])
def test_attn_mask_on_a_mixed_batch(orc, torch_dev, pkg, per_head, cache_prefill):
    """The optional attn_mask input: additive fp16, [T, C] or [num_heads, T, C], element
    [.., seqstarts[b] + i, kvstarts[b] + j]; decode and prefill sequences in one call, split-k forced on a long
    decode sequence, prefill with and without the INT8 cache (history included)."""
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=8, num_kv_heads=2, head_dim=128, n_decode=3, kv_dist="list", kv_list=(40, 700, 17),
                 n_prefill=3, seed=35)
    hc = workloads.host_case(spec)
    idx = workloads.make_index([40, 700, 17], [100, 64, 150], prefill_hist=[0, 90, 31] if cache_prefill else None)
    hc = _case_with_index(hc, idx, spec)
    mask = _random_mask(np.random.default_rng(36), idx, heads=8 if per_head else None, cols_extra=16 if per_head else 0)
    run_case(orc, torch_dev, hc, cache_prefill=cache_prefill, attn_mask=mask, split_k=2)


def test_attn_mask_head_dim_64_and_a_narrow_mask_is_reported(orc, torch_dev, pkg):
    import torch
    from ppl_nn_b200 import ops, workloads
    spec = _spec(num_heads=8, num_kv_heads=8, head_dim=64, n_decode=4, kv_dist="list", kv_list=(17, 64, 130, 255),
                 n_prefill=1, seed=37)
    hc = workloads.host_case(spec)
    idx = workloads.make_index([17, 64, 130, 255], [70])
    hc = _case_with_index(hc, idx, spec)
    mask = _random_mask(np.random.default_rng(38), idx)
    err, op = run_case(orc, torch_dev, hc, attn_mask=mask)
    # a mask with too few columns for kvstarts: nothing is read past its rows' ends, and the status word says so
    dev = torch_dev
    narrow = np.ascontiguousarray(mask[:, :256])
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, 8, 64)
    out = op.forward(_t(hc.query, dev), _t(hc.current_key, dev), _t(hc.current_value, dev), _t(idx.seqstarts, dev),
                     _t(idx.kvstarts, dev), _t(idx.cachestarts, dev), _t(idx.start_pos, dev), idx.decoding_batches,
                     idx.max_seqlen, idx.max_kvlen, torch.zeros(cshape, dtype=torch.int8, device=dev),
                     torch.zeros(sshape, dtype=torch.float16, device=dev), attn_mask=_t(narrow, dev))
    assert op.device_status() & 16
    assert bool(torch.isfinite(out.float()).all())


def test_smoke_entry_point(torch_dev):
    import __graft_entry__ as entry
    entry.smoke()


def test_kv_head_shards_concatenate_to_the_unsharded_output(orc, torch_dev, pkg):
    """The multi-GPU decomposition, rank by rank on one GPU: every rank's call on its kv-head shard
    (own cache, replicated index tensors), outputs concatenated along the head axis.  With split-k off
    every (sequence, head) is computed by the same instruction sequence as in the unsharded call, so
    the result is bit-identical; with the stream-k split the cut points move, so it is compared within
    the tolerance."""
    import torch
    from ppl_nn_b200 import ops, sharding, workloads
    spec = workloads.scaled(workloads.SPECS["cfg4_llama70b_decode"], seqs=24 / 512, length=0.2)
    full = workloads.host_case(spec)
    idx, hidx = full.index, full.hist_index
    Hq, Hkv, Dh = spec.num_heads, spec.num_kv_heads, spec.head_dim
    dev = torch_dev

    def run(q, ck, cv, hk, hv, hq, hkv, split_k):
        cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, hkv, Dh)
        cache = torch.zeros(cshape, dtype=torch.int8, device=dev)
        scale = torch.zeros(sshape, dtype=torch.float16, device=dev)
        kvc = ops.KeyValueCache(ops.KeyValueCacheParam(num_layer=1, layer_idx=0, quant_bit=8))
        kvc.forward(_t(hk, dev), _t(hv, dev), _t(hidx.seqstarts, dev), _t(hidx.kvstarts, dev),
                    _t(hidx.cachestarts, dev), _t(hidx.start_pos, dev), hidx.max_seqlen, hidx.max_kvlen, cache, scale,
                    total_kv=0)
        op = ops.MultiHeadCacheAttention(
            ops.MultiHeadCacheAttentionParam(num_heads=hq, num_kv_heads=hkv, head_dim=Dh, num_layer=1, layer_idx=0,
                                             quant_bit=8), ops.EngineConfig(specify_decoding_attn_split_k=split_k))
        out = op.forward(_t(q, dev), _t(ck, dev), _t(cv, dev), _t(idx.seqstarts, dev), _t(idx.kvstarts, dev),
                         _t(idx.cachestarts, dev), _t(idx.start_pos, dev), idx.decoding_batches, idx.max_seqlen,
                         idx.max_kvlen, cache, scale)
        assert op.device_status() == 0
        return out.cpu().numpy()

    for split_k in (0, 1):
        whole = run(full.query, full.current_key, full.current_value, full.hist_key, full.hist_value, Hq, Hkv, split_k)
        for world in (2, 8):
            parts = []
            for rank in range(world):
                qs, kvs = sharding.head_shard(Hq, Hkv, rank, world)
                lq, lk, lv = sharding.shard_call(full.query, full.current_key, full.current_value, Hq, Hkv, rank, world)
                parts.append(run(lq, lk, lv, np.ascontiguousarray(full.hist_key[:, kvs]),
                                 np.ascontiguousarray(full.hist_value[:, kvs]), qs.stop - qs.start,
                                 kvs.stop - kvs.start, split_k))
            joined = np.concatenate(parts, axis=1)
            if split_k == 0:
                np.testing.assert_array_equal(joined.view(np.uint16), whole.view(np.uint16))
            else:
                err = np.abs(joined.astype(np.float32) - whole.astype(np.float32))
                assert err.max() <= MAX_ABS and err.mean() <= MEAN_ABS


def _two_gpu_rank(rank, world, port, result_dir):
    import os
    import sys
    from pathlib import Path
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    root = Path(__file__).resolve().parent.parent
    sys.path.insert(0, str(root))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    from ppl_nn_b200 import ops, sharding, workloads
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        spec = workloads.scaled(workloads.SPECS["cfg4_llama70b_decode"], seqs=16 / 512, length=0.1)
        full = workloads.host_case(spec)  # same seed on every rank: identical full tensors
        idx, hidx = full.index, full.hist_index
        Hq, Hkv, Dh = spec.num_heads, spec.num_kv_heads, spec.head_dim
        qs, kvs = sharding.head_shard(Hq, Hkv, rank, world)
        lq, lk, lv = sharding.shard_call(full.query, full.current_key, full.current_value, Hq, Hkv, rank, world)
        hq, hkv = qs.stop - qs.start, kvs.stop - kvs.start
        cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, hkv, Dh)
        cache = torch.zeros(cshape, dtype=torch.int8, device=dev)
        scale = torch.zeros(sshape, dtype=torch.float16, device=dev)

        def t(a):
            return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

        kvc = ops.KeyValueCache(ops.KeyValueCacheParam(num_layer=1, layer_idx=0, quant_bit=8))
        kvc.forward(t(full.hist_key[:, kvs]), t(full.hist_value[:, kvs]), t(hidx.seqstarts), t(hidx.kvstarts),
                    t(hidx.cachestarts), t(hidx.start_pos), hidx.max_seqlen, hidx.max_kvlen, cache, scale, total_kv=0)
        op = ops.MultiHeadCacheAttention(ops.MultiHeadCacheAttentionParam(num_heads=hq, num_kv_heads=hkv, head_dim=Dh,
                                                                         num_layer=1, layer_idx=0, quant_bit=8))
        out = op.forward(t(lq), t(lk), t(lv), t(idx.seqstarts), t(idx.kvstarts), t(idx.cachestarts), t(idx.start_pos),
                         idx.decoding_batches, idx.max_seqlen, idx.max_kvlen, cache, scale)
        gathered = sharding.gather_heads(out, world)  # NCCL all-gather, verification only
        torch.cuda.synchronize(dev)
        if rank == 0:
            np.save(os.path.join(result_dir, "gathered.npy"), gathered.cpu().numpy())
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpus_nccl_gather_matches_the_oracle(orc, torch_dev, pkg, tmp_path):
    """Real ranks on real GPUs (needs two of them): each rank runs its shard, NCCL gathers the heads,
    and the gathered tensor is checked against the oracle on the unsharded problem."""
    import socket
    import torch
    import torch.multiprocessing as mp
    from ppl_nn_b200 import workloads
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on the node")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_two_gpu_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got = np.load(tmp_path / "gathered.npy").astype(np.float32)
    spec = workloads.scaled(workloads.SPECS["cfg4_llama70b_decode"], seqs=16 / 512, length=0.1)
    full = workloads.host_case(spec)
    idx, hidx = full.index, full.hist_index
    Hq, Hkv, Dh = spec.num_heads, spec.num_kv_heads, spec.head_dim
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
    cache = np.zeros(cshape, dtype=np.int8)
    scale = np.zeros(sshape, dtype=np.float16)
    kw = dict(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, max_tokens=idx.max_tokens)
    orc.kv_append(orc.desc(decoding_batches=0, **kw), full.hist_key, full.hist_value, hidx.seqstarts, hidx.cachestarts,
                  hidx.start_pos, cache, scale)
    want = orc.mhca(orc.desc(decoding_batches=idx.decoding_batches, **kw), full.query, full.current_key,
                    full.current_value, idx.seqstarts, idx.cachestarts, idx.start_pos, cache, scale).astype(np.float32)
    err = np.abs(got - want)
    assert got.shape == want.shape and err.max() <= MAX_ABS and err.mean() <= MEAN_ABS
