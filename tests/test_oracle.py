"""The CPU oracle checked against itself: hand-derived known answers of the quantiser, the numpy
twin, structural properties, and the committed golden outputs of the tiny configuration.

The reference tree holds no golden vector for this path, so the known answers here are derived by
hand from the published formula (INT8 symmetric, group 8, fp16 scale = absmax/127) and the golden
files under tests/golden/ are the oracle's own output, kept as regression pins."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"


def h16(vals):
    return np.array(vals, dtype=np.float16)


# (input group, expected codes, expected scale) -- each derivable with pencil and paper
KNOWN = [
    # absmax 127 -> scale exactly 1; ties go to even: 63.5 -> 64, 0.5 -> 0, 2.5 -> 2, -1.5 -> -2
    ([127, 0, -127, 63.5, 1, -1, 0.5, 64], [127, 0, -127, 64, 1, -1, 0, 64], 1.0),
    ([127, 2.5, -1.5, 3.5, -2.5, 126.5, -126.5, 0.25], [127, 2, -2, 4, -2, 126, -126, 0], 1.0),
    # absmax 254 -> scale 2
    ([254, 1, 3, 5, -3, -254, 7, 2], [127, 0, 2, 2, -2, -127, 4, 1], 2.0),
    # all zero -> scale 0 -> codes 0; negative zero is still zero
    ([0, 0, 0, 0, 0, 0, 0, 0], [0] * 8, 0.0),
    ([-0.0, 0, -0.0, 0, 0, 0, 0, 0], [0] * 8, 0.0),
    # one element: it maps to +-127, everything else to 0
    ([0, 0, 0, -63.5, 0, 0, 0, 0], [0, 0, 0, -127, 0, 0, 0, 0], 0.5),
]


@pytest.mark.parametrize("x,codes,scale", KNOWN)
def test_quantiser_known_answers(orc, oracle_mod, x, codes, scale):
    c, s = orc.quant_groups(h16(x))
    assert c.tolist() == codes
    assert float(s[0]) == scale
    c2, s2 = oracle_mod.np_quant_groups(h16(x))
    assert c2.tolist() == codes and float(s2[0]) == scale


def test_fp16_conversion_matches_numpy_everywhere(orc):
    # all 65536 half patterns -> float exactly as numpy does
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = np.array([orc.half_to_float(int(h)) for h in allh[::7]], dtype=np.float32)
    nan = np.isnan(ref[::7])
    np.testing.assert_array_equal(got[~nan].view(np.uint32), ref[::7][~nan].view(np.uint32))
    assert np.all(np.isnan(got[nan]))  # NaN stays NaN (the payload's quiet bit is not compared)
    # float -> half round-to-nearest-even on a spread of magnitudes, ties, subnormals, overflow
    rng = np.random.default_rng(0)
    f = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 4000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001, 2.0 ** -14,
                  (1 + 2.0 ** -11), (1 + 3 * 2.0 ** -11), 6.1e-5, 5.96e-8, 3e-8, np.inf, -np.inf], dtype=np.float32)])
    want = f.astype(np.float16).view(np.uint16)
    got = np.array([orc.float_to_half(float(v)) for v in f], dtype=np.uint16)
    np.testing.assert_array_equal(got, want)


def test_c_quantiser_equals_numpy_twin_bit_for_bit(orc, oracle_mod):
    rng = np.random.default_rng(7)
    x = (rng.standard_normal((3000, 8)) * (10.0 ** rng.integers(-7, 5, (3000, 1)))).astype(np.float16)
    x[::50, 3] = np.float16(65504)
    x[1::50, 5] = np.float16(-65504)
    x[2::50] = np.float16(6e-8)      # subnormal halves: the scale rounds to zero
    x[3::50, :] = np.float16(0.37)   # all equal
    x[4::50, 2] = np.float16("nan")
    x[5::50, 6] = np.float16("inf")
    c1, s1 = orc.quant_groups(x)
    c2, s2 = oracle_mod.np_quant_groups(x)
    np.testing.assert_array_equal(c1, c2)
    np.testing.assert_array_equal(s1.view(np.uint16), s2.reshape(s1.shape).view(np.uint16))


def test_quantiser_properties(oracle_mod):
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((5000, 8)) * (10.0 ** rng.integers(-3, 4, (5000, 1)))).astype(np.float16)
    c, s = oracle_mod.np_quant_groups(x)
    assert c.min() >= -127 and c.max() <= 127
    deq = oracle_mod.np_dequant(c, s.reshape(-1, 1))
    sf = s.astype(np.float32).reshape(-1, 1)
    xf = x.astype(np.float32)
    # round trip within half a step (plus the effect of rounding the scale to fp16), wherever the
    # scale is a normal half; a subnormal scale is coarser and the absmax element is clamped to 127
    normal = (sf >= 2.0 ** -14).ravel()
    assert normal.sum() > 4000
    assert np.all((np.abs(deq - xf) <= 0.5 * sf + np.abs(xf) * 2.0 ** -10)[normal])
    # the absmax element maps to +-127
    am = np.abs(xf).argmax(axis=1)
    assert np.all((np.abs(c[np.arange(c.shape[0]), am]) == 127)[normal])


def _tiny_case(pkg, orc):
    from ppl_nn_b200 import workloads
    hc = workloads.host_case(workloads.SPECS["cfg1_tiny"])
    idx, hidx = hc.index, hc.hist_index
    Hq, Hkv, Dh = hc.num_heads, hc.num_kv_heads, hc.spec.head_dim
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
    cache = np.zeros(cshape, dtype=np.int8)
    scale = np.zeros(sshape, dtype=np.float16)
    d0 = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, decoding_batches=0,
                  max_tokens=idx.max_tokens)
    orc.kv_append(d0, hc.hist_key, hc.hist_value, hidx.seqstarts, hidx.cachestarts, hidx.start_pos, cache, scale)
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, decoding_batches=idx.decoding_batches,
                 max_tokens=idx.max_tokens)
    out = orc.mhca(d, hc.query, hc.current_key, hc.current_value, idx.seqstarts, idx.cachestarts, idx.start_pos,
                   cache, scale)
    return hc, d, cache, scale, out


def test_tiny_config_matches_golden(pkg, orc):
    hc, d, cache, scale, out = _tiny_case(pkg, orc)
    meta = json.loads((GOLDEN / "cfg1_tiny.json").read_text())
    assert hc.index.kvlens[:4].tolist() == [17, 64, 130, 255]
    assert hashlib.sha256(cache.tobytes()).hexdigest() == meta["cache_sha256"]
    assert hashlib.sha256(scale.tobytes()).hexdigest() == meta["scale_sha256"]
    want = np.fromfile(GOLDEN / meta["attn_output_file"], dtype=np.float16).reshape(out.shape)
    np.testing.assert_allclose(out.astype(np.float32), want.astype(np.float32), atol=1e-3, rtol=0)


def test_attention_equals_numpy_twin(pkg, orc, oracle_mod):
    hc, d, cache, scale, out = _tiny_case(pkg, orc)
    idx = hc.index
    deq = oracle_mod.np_dequant(cache, scale)  # (MaxT, 1, 2, H, Dh)
    for b in range(idx.batch):
        n = int(idx.kvlens[b])
        rows = slice(int(idx.cachestarts[b]), int(idx.cachestarts[b]) + n)
        for h in (0, 3, 7):
            q = hc.query[idx.seqstarts[b], h].astype(np.float32)
            ref = oracle_mod.np_attention_one(q, deq[rows, 0, 0, h], deq[rows, 0, 1, h])
            np.testing.assert_allclose(out[idx.seqstarts[b], h].astype(np.float32), ref, atol=1e-3, rtol=1e-3)


def test_gather_dequant_round_trip(pkg, orc, oracle_mod):
    hc, d, cache, scale, _ = _tiny_case(pkg, orc)
    idx = hc.index
    key, value = orc.kv_gather_dequant(d, idx.kvstarts, idx.cachestarts, cache, scale)
    assert key.shape == (int(idx.kvstarts[-1]), hc.num_kv_heads, hc.spec.head_dim)
    # the last row of every sequence is this step's token: dequantised it is within half a step
    for b in range(idx.batch):
        last = int(idx.kvstarts[b + 1]) - 1
        x = hc.current_key[idx.seqstarts[b]].astype(np.float32)
        c, s = oracle_mod.np_quant_groups(hc.current_key[idx.seqstarts[b]])
        np.testing.assert_array_equal(key[last].astype(np.float32),
                                      oracle_mod.np_dequant(c, s).astype(np.float16).astype(np.float32))
        assert np.all(np.abs(key[last].astype(np.float32) - x) <= 0.51 * np.repeat(s.astype(np.float32), 8, -1) + 1e-3)


def test_layout3_and_paged_give_the_same_attention(pkg, orc):
    """cache_layout 3 and the paged mode are pure re-addressings: same codes, same output."""
    from ppl_nn_b200 import workloads
    spec = workloads.SPECS["cfg1_tiny"]
    outs = []
    for layout, page in ((0, 0), (3, 0), (0, 16), (3, 32)):
        hc = workloads.host_case(spec, page_size=page)
        idx, hidx = hc.index, hc.hist_index
        cshape, sshape = workloads.cache_shapes(layout, idx.max_tokens, 2, hc.num_kv_heads, spec.head_dim)
        cache = np.zeros(cshape, dtype=np.int8)
        scale = np.zeros(sshape, dtype=np.float16)
        kw = dict(num_heads=hc.num_heads, num_kv_heads=hc.num_kv_heads, head_dim=spec.head_dim, batch=idx.batch,
                  max_tokens=idx.max_tokens, num_layer=2, layer_idx=1, cache_layout=layout,
                  cache_mode=1 if page else 0, page_size=page or 128,
                  cachestart_stride_b=idx.cachestarts.shape[1] if page else 0)
        orc.kv_append(orc.desc(decoding_batches=0, **kw), hc.hist_key, hc.hist_value, hidx.seqstarts, hidx.cachestarts,
                      hidx.start_pos, cache, scale)
        outs.append(orc.mhca(orc.desc(decoding_batches=idx.decoding_batches, **kw), hc.query, hc.current_key,
                             hc.current_value, idx.seqstarts, idx.cachestarts, idx.start_pos, cache, scale))
        # layer 0 was never written
        if layout == 0:
            assert not cache[:, 0].any()
        else:
            assert not cache[0].any()
    for o in outs[1:]:
        np.testing.assert_array_equal(o.view(np.uint16), outs[0].view(np.uint16))


def test_prefill_is_causal_and_gqa_maps_heads(pkg, orc, oracle_mod):
    from dataclasses import replace
    from ppl_nn_b200 import workloads
    spec = replace(workloads.SPECS["cfg1_tiny"], num_heads=8, num_kv_heads=2, n_decode=0, kv_list=(), n_prefill=2,
                   pf_lo=5, pf_hi=9, seed=5)
    hc = workloads.host_case(spec)
    idx = hc.index
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, 2, spec.head_dim)
    cache = np.zeros(cshape, dtype=np.int8)
    scale = np.zeros(sshape, dtype=np.float16)
    d = orc.desc(num_heads=8, num_kv_heads=2, head_dim=spec.head_dim, batch=idx.batch, decoding_batches=0,
                 max_tokens=idx.max_tokens)
    out = orc.mhca(d, hc.query, hc.current_key, hc.current_value, idx.seqstarts, idx.cachestarts, idx.start_pos,
                   cache, scale)
    # fp16 K/V of this call, no history: token i sees tokens 0..i of its own sequence
    for b in range(idx.batch):
        s0 = int(idx.seqstarts[b])
        for i in range(int(idx.seqlens[b])):
            for h in (0, 3, 4, 7):
                k = hc.current_key[s0:s0 + i + 1, h // 4].astype(np.float32)
                v = hc.current_value[s0:s0 + i + 1, h // 4].astype(np.float32)
                ref = oracle_mod.np_attention_one(hc.query[s0 + i, h].astype(np.float32), k, v)
                np.testing.assert_allclose(out[s0 + i, h].astype(np.float32), ref, atol=1e-3, rtol=1e-3)
    # with enable_cache_prefill the same call reads the quantised cache instead
    d2 = orc.desc(num_heads=8, num_kv_heads=2, head_dim=spec.head_dim, batch=idx.batch, decoding_batches=0,
                  max_tokens=idx.max_tokens, enable_cache_prefill=1)
    out2 = orc.attention(d2, hc.query, hc.current_key, hc.current_value, idx.seqstarts, idx.cachestarts, idx.start_pos,
                         cache, scale)
    assert np.abs(out2.astype(np.float32) - out.astype(np.float32)).max() < 0.05  # quantisation noise only
    assert not np.array_equal(out2, out)


# ---- an implementation the oracle shares no code with: torch's scaled_dot_product_attention -----------
def _sdpa(q, k, v, causal_offset=None):
    """q [Tq, H, Dh], k/v [Tk, H, Dh] (float32 torch) -> [Tq, H, Dh]; causal_offset: row i sees kv <= i + offset."""
    import torch
    mask = None
    if causal_offset is not None:
        i = torch.arange(q.shape[0])[:, None]
        j = torch.arange(k.shape[0])[None, :]
        mask = j <= i + causal_offset
    o = torch.nn.functional.scaled_dot_product_attention(q.transpose(0, 1)[None].double(), k.transpose(0, 1)[None].double(),
                                                         v.transpose(0, 1)[None].double(), attn_mask=mask)
    return o[0].transpose(0, 1).float()


def test_decode_attention_agrees_with_torch_sdpa(pkg, orc, oracle_mod):
    """The oracle's decode over the INT8 cache against torch SDPA (float64) over the dequantised rows."""
    import torch
    hc, d, cache, scale, out = _tiny_case(pkg, orc)
    idx = hc.index
    deq = torch.from_numpy(oracle_mod.np_dequant(cache, scale).astype(np.float32))  # (MaxT, 1, 2, H, Dh)
    for b in range(idx.batch):
        n = int(idx.kvlens[b])
        r0 = int(idx.cachestarts[b])
        q = torch.from_numpy(hc.query[idx.seqstarts[b]:idx.seqstarts[b] + 1].astype(np.float32))
        ref = _sdpa(q, deq[r0:r0 + n, 0, 0], deq[r0:r0 + n, 0, 1]).numpy()
        got = out[idx.seqstarts[b]:idx.seqstarts[b] + 1].astype(np.float32)
        np.testing.assert_allclose(got, ref, atol=1e-3, rtol=1e-3)  # the oracle rounds its output to fp16


@pytest.mark.parametrize("causal", [True, False])
def test_uncached_attention_agrees_with_torch_sdpa(orc, causal):
    """orc_mha (GQA 4/2 heads, kv longer than q, mask aligned to the end) against torch SDPA (float64)."""
    import torch
    rng = np.random.default_rng(21)
    seqlens, kvlens, Hq, Hkv, Dh = [6, 1, 17], [6, 40, 29], 4, 2, 64
    ss = np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int64)
    ks = np.concatenate([[0], np.cumsum(kvlens)]).astype(np.int64)
    q = rng.standard_normal((int(ss[-1]), Hq, Dh)).astype(np.float16)
    k = rng.standard_normal((int(ks[-1]), Hkv, Dh)).astype(np.float16)
    v = rng.standard_normal((int(ks[-1]), Hkv, Dh)).astype(np.float16)
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=len(seqlens), is_causal=int(causal))
    got = orc.mha(d, q, k, v, ss, ks).astype(np.float32)
    rep = Hq // Hkv
    for b in range(len(seqlens)):
        qq = torch.from_numpy(q[ss[b]:ss[b + 1]].astype(np.float32))
        kk = torch.from_numpy(k[ks[b]:ks[b + 1]].astype(np.float32)).repeat_interleave(rep, dim=1)
        vv = torch.from_numpy(v[ks[b]:ks[b + 1]].astype(np.float32)).repeat_interleave(rep, dim=1)
        ref = _sdpa(qq, kk, vv, causal_offset=(kvlens[b] - seqlens[b]) if causal else None).numpy()
        np.testing.assert_allclose(got[ss[b]:ss[b + 1]], ref, atol=1e-3, rtol=1e-3)


def test_fast_quantiser_path_of_the_cuda_kernels_gives_the_exact_codes(oracle_mod):
    """The CUDA quantiser (csrc/common.cuh::quant_group8) avoids the eight divisions of a group: it multiplies
    by an approximate reciprocal of the scale (1 ulp off at most), rounds with the add-and-subtract of
    1.5 * 2^23, and trusts the result only if the scale is a normal half and every product is further than
    1e-4 from a half-integer; any other group is redone with the true divisions.  Restated here in numpy
    float32 (IEEE, like the device's non-fused operations) with the reciprocal pushed one ulp either way:
    whenever the fast path trusts itself its codes are the codes of the published formula."""
    rng = np.random.default_rng(17)
    magic = np.float32(12582912.0)
    total_fast = 0
    for mode, scale in enumerate([1.0, 1e-3, 300.0, 3e-5, 6e4, None]):
        n = 200_000
        mag = np.float32(scale) if scale is not None else (10.0 ** rng.uniform(-4.5, 4.5, (n, 1))).astype(np.float32)
        x = (rng.standard_normal((n, 8)).astype(np.float32) * mag).astype(np.float16)
        # adversarial half: values at (k + 0.5) * s of their own group's scale
        a0 = np.abs(x.astype(np.float32)).max(axis=1)
        s0 = (a0 / np.float32(127.0)).astype(np.float16).astype(np.float32)
        k = rng.integers(-126, 126, (n, 7)).astype(np.float32) + np.float32(0.5)
        adv = rng.random(n) < 0.5
        x[adv, 1:] = (k[adv] * s0[adv, None]).astype(np.float16)
        codes, scales = oracle_mod.np_quant_groups(x)       # the published formula (exact divisions)
        v = x.astype(np.float32)
        s = scales.astype(np.float32).reshape(n, 1)
        ok = np.isfinite(s[:, 0]) & (s[:, 0] != 0)
        v, s, codes = v[ok], s[ok], codes.reshape(n, 8)[ok]
        with np.errstate(over="ignore", invalid="ignore"):
            r0 = (np.float32(1.0) / s).astype(np.float32)
            for r in (r0, np.nextafter(r0, np.float32(np.inf)), np.nextafter(r0, np.float32(0))):
                qf = (v * r).astype(np.float32)
                u = (qf + magic).astype(np.float32)
                t = (u - magic).astype(np.float32)
                safe = (s[:, 0] >= np.float32(6.103515625e-05)) & (np.abs((qf - t).astype(np.float32)) < np.float32(0.4999)).all(axis=1)
                fast = (u.view(np.uint32) & 0xFF).astype(np.uint8).view(np.int8)
                np.testing.assert_array_equal(fast[safe], codes[safe])
                total_fast += int(safe.sum())
    assert total_fast > 1_000_000  # the fast path is the common case, so the check is not vacuous


def test_scale_by_reciprocal_equals_the_division_for_every_half():
    """The CUDA quantiser computes the group scale as fp16(a * fl(1/127)) instead of fp16(fl(a / 127)).  The
    maximum a is itself an fp16 number, so the claim can be checked for every one of them: the two agree bit
    for bit, also with the constant one ulp off either way (the margin the argument in common.cuh gives)."""
    a = np.arange(0, 0x7C01, dtype=np.uint16).view(np.float16).astype(np.float32)  # every non-negative half, +inf
    with np.errstate(over="ignore"):
        ref = (a / np.float32(127.0)).astype(np.float32).astype(np.float16).view(np.uint16)
        r = np.float32(1.0) / np.float32(127.0)
        for c in (r, np.nextafter(r, np.float32(1)), np.nextafter(r, np.float32(0))):
            got = (a * c).astype(np.float32).astype(np.float16).view(np.uint16)
            np.testing.assert_array_equal(got, ref)


def test_integer_dot_scores_of_the_decode_kernel(oracle_mod):
    """With one query head per kv head the decode kernel quantises the query row to int16 with one fp32 scale
    per 8-channel group and takes a group's partial score as the exact integer dot product of codes and
    quantised query times key scale times query scale (csrc/decode_splitk.cu, KDOT).  Restated in numpy: the
    score differs from the exactly dequantised one by at most 2^-16 of sum_g s_g * max|q_g| * sum|c|, and in
    practice by a few 1e-6 relative to the score's own scale."""
    rng = np.random.default_rng(23)
    T, Dh = 512, 128
    k = rng.standard_normal((T, Dh)).astype(np.float32)
    k[:, ::16] *= 8.0  # outlier channels, as in the LLaMA-2-7B workload
    codes, scales = oracle_mod.np_quant_groups(k.astype(np.float16).reshape(-1, 8))
    c = codes.reshape(T, Dh // 8, 8).astype(np.int64)
    s = scales.astype(np.float32).reshape(T, Dh // 8)
    q = (rng.standard_normal(Dh) * rng.choice([0.01, 1.0, 30.0], Dh)).astype(np.float16).astype(np.float32)
    qg = q.reshape(Dh // 8, 8)
    amax = np.abs(qg).max(axis=1)
    inv = np.where(amax > 0, np.float32(32767.0) / amax, 0).astype(np.float32)
    qs = (amax * np.float32(1.0 / 32767.0)).astype(np.float32)
    qi = np.rint((qg * inv[:, None]).astype(np.float32)).astype(np.int64)
    assert np.abs(qi).max() <= 32767
    idot = (c * qi[None]).sum(axis=2)                                  # exact in int32 on the device
    assert np.abs(idot).max() < 2 ** 31
    got = (idot.astype(np.float32) * (s * qs[None]).astype(np.float32)).astype(np.float64).sum(axis=1)
    want = ((c * s[:, :, None].astype(np.float64)) * qg[None].astype(np.float64)).sum(axis=(1, 2))
    bound = (s.astype(np.float64) * amax[None] * np.abs(c).sum(axis=2)).sum(axis=1) * 2.0 ** -16 + 1e-6 * np.abs(want).max()
    assert (np.abs(got - want) <= bound).all()
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()


@pytest.mark.parametrize("cache_prefill", [False, True])
def test_cached_operator_mask_matches_numpy(pkg, orc, oracle_mod, cache_prefill):
    """attn_mask in orc_mhca against numpy over the dequantised rows: decode rows read the cache from position 0,
    prefill rows read this call's fp16 K/V (mask columns start at start_pos) or, with enable_cache_prefill, the
    cache (mask columns start at 0)."""
    from ppl_nn_b200 import workloads
    rng = np.random.default_rng(9)
    Hq, Hkv, Dh = 4, 2, 64
    idx = workloads.make_index([9, 30], [6, 11], prefill_hist=[0, 5] if cache_prefill else [0, 5])
    T, KV = idx.total_tokens, int(idx.kvstarts[-1])
    q = rng.standard_normal((T, Hq, Dh)).astype(np.float16)
    ck = rng.standard_normal((T, Hkv, Dh)).astype(np.float16)
    cv = rng.standard_normal((T, Hkv, Dh)).astype(np.float16)
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
    cache = rng.integers(-127, 128, size=cshape, dtype=np.int8)
    scale = rng.uniform(0.004, 0.02, size=sshape).astype(np.float16)
    mask = (rng.standard_normal((T, (KV + 7) // 8 * 8)) * 0.5).astype(np.float16)
    mask[rng.random(mask.shape) < 0.2] = -np.inf
    d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, decoding_batches=2,
                 max_tokens=idx.max_tokens, enable_cache_prefill=int(cache_prefill))
    got = orc.mhca(d, q, ck, cv, idx.seqstarts, idx.cachestarts, idx.start_pos, cache, scale, kvstarts=idx.kvstarts,
                   attn_mask=mask).astype(np.float32)
    deq = oracle_mod.np_dequant(cache[:, 0], scale[:, 0])  # [rows, 2, Hkv, Dh] after the append
    for b in range(idx.batch):
        s0, k0, c0, sp = int(idx.seqstarts[b]), int(idx.kvstarts[b]), int(idx.cachestarts[b]), int(idx.start_pos[b])
        from_cache = b < 2 or cache_prefill
        for i in range(int(idx.seqlens[b])):
            n = sp + i + 1 if from_cache else i + 1
            for h in range(Hq):
                if from_cache:
                    k, v = deq[c0:c0 + n, 0, h // 2], deq[c0:c0 + n, 1, h // 2]
                    mrow = mask[s0 + i, k0:k0 + n]
                else:
                    k = ck[s0:s0 + n, h // 2].astype(np.float32)
                    v = cv[s0:s0 + n, h // 2].astype(np.float32)
                    mrow = mask[s0 + i, k0 + sp:k0 + sp + n]
                want = oracle_mod.np_attention_one(q[s0 + i, h].astype(np.float32), k, v, mrow)
                assert np.abs(got[s0 + i, h] - want).max() <= 2e-3, (b, i, h)
