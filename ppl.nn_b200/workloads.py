"""Seeded synthetic workloads: the five benchmark configurations and scaled-down variants.

Every workload is one call of MultiHeadCacheAttention on one transformer layer: ``n_decode``
decode sequences (one new token each, ``start_pos = kvlen - 1`` tokens of history in the cache)
followed by ``n_prefill`` prefill sequences, with the ragged index tensors built the way ppl.nn's
own driver builds them (tools/benchmark_llama/generation_state.cc:60-192): seqstarts and kvstarts
are prefix sums, cachestarts is the running sum of per-sequence cache capacities.

Two builders:
  * ``host_case``   numpy arrays, including the fp16 history, for cases small enough for a CPU check;
  * ``device_case`` torch CUDA tensors for full-size runs; the history is generated on the device in
                    slabs and written into the INT8 cache by the library's own append kernel.
Values follow the configuration text: N(0,1) everywhere; ``outlier_k`` multiplies every 16th K
channel by 8; ``peaked`` adds +6 to all channels of ~1% of the key positions.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace

import numpy as np


@dataclass(frozen=True)
class Spec:
    name: str
    num_heads: int
    num_kv_heads: int
    head_dim: int
    n_decode: int
    kv_lo: int
    kv_hi: int
    kv_dist: str = "uniform"  # "uniform" | "loguniform" | "list"
    kv_list: tuple = ()
    n_prefill: int = 0
    pf_lo: int = 0
    pf_hi: int = 0
    seed: int = 0
    outlier_k: bool = False
    peaked: bool = False
    is_causal: bool = True
    pf_skip: int = 0  # decode lengths drawn and dropped before the prompts (the prompts of a mixed spec on their own)


SPECS = {
    # Tiny CPU-runnable ragged decode
    "cfg1_tiny": Spec("cfg1_tiny", 8, 8, 64, 4, 17, 255, "list", (17, 64, 130, 255), seed=0),
    # LLaMA-2-7B attention layer, pure decode
    "cfg2_llama7b_decode": Spec("cfg2_llama7b_decode", 32, 32, 128, 256, 128, 4096, seed=1, outlier_k=True),
    # LLaMA-3-8B attention layer, mixed continuous-batching step
    "cfg3_llama8b_mixed": Spec("cfg3_llama8b_mixed", 32, 8, 128, 248, 256, 8192, n_prefill=8, pf_lo=512, pf_hi=2048,
                               seed=2),
    # the prefill half of the mixed step alone (for the tensor-core roofline of the prefill kernel)
    "cfg3_prefill_only": Spec("cfg3_prefill_only", 32, 8, 128, 0, 256, 8192, n_prefill=8, pf_lo=512, pf_hi=2048, seed=2,
                              pf_skip=248),
    # the same layer with 16 prompts of 4096 tokens: the steady state of the prefill kernel (not a BASELINE config)
    "prefill_16x4096": Spec("prefill_16x4096", 32, 8, 128, 0, 1, 1, n_prefill=16, pf_lo=4096, pf_hi=4096, seed=5),
    # LLaMA-2-70B attention layer, large-batch decode
    "cfg4_llama70b_decode": Spec("cfg4_llama70b_decode", 64, 8, 128, 512, 64, 8192, "loguniform", seed=3),
    # Long-context split-k stress
    "cfg5_longctx": Spec("cfg5_longctx", 32, 8, 128, 16, 32768, 131072, seed=4, peaked=True),
}


def scaled(spec: Spec, seqs: float = 1.0, length: float = 1.0) -> Spec:
    """A smaller workload of the same shape: fewer sequences and/or shorter lengths."""
    def sc(v, f, lo=1):
        return max(lo, int(round(v * f)))
    return replace(spec, name=f"{spec.name}@{seqs:g}x{length:g}",
                   n_decode=sc(spec.n_decode, seqs, 0 if spec.n_decode == 0 else 1),
                   n_prefill=sc(spec.n_prefill, seqs, 0 if spec.n_prefill == 0 else 1),
                   kv_lo=sc(spec.kv_lo, length), kv_hi=sc(spec.kv_hi, length),
                   kv_list=tuple(sc(v, length) for v in spec.kv_list),
                   pf_lo=sc(spec.pf_lo, length, 0), pf_hi=sc(spec.pf_hi, length, 0))


@dataclass
class Index:
    """Host-side ragged index tensors of one call (all int64 numpy) plus the host scalars."""
    seqstarts: np.ndarray
    kvstarts: np.ndarray
    cachestarts: np.ndarray
    start_pos: np.ndarray
    seqlens: np.ndarray
    decoding_batches: int
    max_seqlen: int
    max_kvlen: int
    total_tokens: int
    max_tokens: int
    page_size: int = 0  # > 0: cachestarts is [batch, max_pages] (cache_mode 1)

    @property
    def batch(self) -> int:
        return int(self.start_pos.shape[0])

    @property
    def kvlens(self) -> np.ndarray:
        return self.start_pos + self.seqlens


def draw_lengths(spec: Spec):
    rng = np.random.default_rng(spec.seed)
    if spec.kv_dist == "list":
        kv = np.array(list(spec.kv_list)[: spec.n_decode] or [], dtype=np.int64)
        if kv.size < spec.n_decode:  # scaled variants may ask for more/less than the list holds
            kv = np.resize(kv, spec.n_decode)
    elif spec.kv_dist == "loguniform":
        kv = np.exp(rng.uniform(np.log(spec.kv_lo), np.log(spec.kv_hi), spec.n_decode)).round().astype(np.int64)
        kv = np.clip(kv, spec.kv_lo, spec.kv_hi)
    else:
        kv = rng.integers(spec.kv_lo, spec.kv_hi + 1, spec.n_decode).astype(np.int64)
        if spec.pf_skip:
            rng.integers(spec.kv_lo, spec.kv_hi + 1, spec.pf_skip)
    pf = rng.integers(spec.pf_lo, spec.pf_hi + 1, spec.n_prefill).astype(np.int64) if spec.n_prefill else \
        np.zeros(0, dtype=np.int64)
    return kv, pf


def make_index(decode_kvlens, prefill_lens, prefill_hist=None, page_size: int = 0, slack_rows: int = 0) -> Index:
    """Decode sequences first (seqlen 1, start_pos = kvlen - 1), then prefill sequences."""
    decode_kvlens = np.asarray(decode_kvlens, dtype=np.int64)
    prefill_lens = np.asarray(prefill_lens, dtype=np.int64)
    if prefill_hist is None:
        prefill_hist = np.zeros_like(prefill_lens)
    seqlens = np.concatenate([np.ones_like(decode_kvlens), prefill_lens])
    start_pos = np.concatenate([decode_kvlens - 1, np.asarray(prefill_hist, dtype=np.int64)])
    kvlens = start_pos + seqlens
    seqstarts = np.concatenate([[0], np.cumsum(seqlens)]).astype(np.int64)
    kvstarts = np.concatenate([[0], np.cumsum(kvlens)]).astype(np.int64)
    if page_size > 0:
        pages = (kvlens + page_size - 1) // page_size
        max_pages = int(pages.max()) if pages.size else 1
        total_pages = int(pages.sum())
        # hand pages out in a shuffled order so that a sequence's pages are not contiguous
        order = np.random.default_rng(12345).permutation(total_pages).astype(np.int64)
        cachestarts = np.zeros((kvlens.size, max_pages), dtype=np.int64)
        k = 0
        for b in range(kvlens.size):
            n = int(pages[b])
            cachestarts[b, :n] = order[k:k + n] * page_size
            k += n
        max_tokens = total_pages * page_size + slack_rows
    else:
        cachestarts = np.concatenate([[0], np.cumsum(kvlens)[:-1]]).astype(np.int64) if kvlens.size else \
            np.zeros(0, dtype=np.int64)
        max_tokens = int(kvlens.sum()) + slack_rows
    return Index(seqstarts=seqstarts, kvstarts=kvstarts, cachestarts=cachestarts, start_pos=start_pos.astype(np.int64),
                 seqlens=seqlens.astype(np.int64), decoding_batches=int(decode_kvlens.size),
                 max_seqlen=int(seqlens.max()) if seqlens.size else 0, max_kvlen=int(kvlens.max()) if kvlens.size else 0,
                 total_tokens=int(seqlens.sum()), max_tokens=max(int(max_tokens), 1), page_size=page_size)


def index_for(spec: Spec, page_size: int = 0) -> Index:
    kv, pf = draw_lengths(spec)
    return make_index(kv, pf, page_size=page_size)


# ------------------------------------------------------------------------------------------------
# values
# ------------------------------------------------------------------------------------------------

def _np_kv(rng, rows, heads, dim, spec: Spec, is_key: bool) -> np.ndarray:
    x = rng.standard_normal((rows, heads, dim), dtype=np.float32)
    if is_key and spec.outlier_k:
        x[:, :, ::16] *= 8.0
    if is_key and spec.peaked and rows > 0:
        hot = rng.random(rows) < 0.01
        x[hot] += 6.0
    return x.astype(np.float16)


@dataclass
class HostCase:
    spec: Spec
    index: Index
    num_kv_heads: int  # heads of this shard
    num_heads: int
    query: np.ndarray
    current_key: np.ndarray
    current_value: np.ndarray
    hist_key: np.ndarray    # [sum(start_pos), Hkv, Dh]: history rows, sequence after sequence
    hist_value: np.ndarray
    hist_index: Index = field(default=None)  # the call that appends the history (start_pos 0)


def host_case(spec: Spec, page_size: int = 0, rank: int = 0, world: int = 1, prefill_hist=None) -> HostCase:
    """Everything in numpy; use only for workloads whose history fits comfortably in host memory."""
    kv, pf = draw_lengths(spec)
    idx = make_index(kv, pf, prefill_hist=prefill_hist, page_size=page_size)
    hkv, hq = spec.num_kv_heads // world, spec.num_heads // world
    rng = np.random.default_rng([spec.seed, 1000 + rank])
    T = idx.total_tokens
    q = rng.standard_normal((T, hq, spec.head_dim), dtype=np.float32).astype(np.float16)
    ck = _np_kv(rng, T, hkv, spec.head_dim, spec, True)
    cv = _np_kv(rng, T, hkv, spec.head_dim, spec, False)
    hist_rows = int(idx.start_pos.sum())
    hk = _np_kv(rng, hist_rows, hkv, spec.head_dim, spec, True)
    hv = _np_kv(rng, hist_rows, hkv, spec.head_dim, spec, False)
    # the call that writes the history: every sequence "prefills" its start_pos tokens at position 0
    hist = Index(seqstarts=np.concatenate([[0], np.cumsum(idx.start_pos)]).astype(np.int64),
                 kvstarts=np.concatenate([[0], np.cumsum(idx.start_pos)]).astype(np.int64),
                 cachestarts=idx.cachestarts, start_pos=np.zeros_like(idx.start_pos), seqlens=idx.start_pos.copy(),
                 decoding_batches=0, max_seqlen=int(idx.start_pos.max()) if idx.batch else 0,
                 max_kvlen=int(idx.start_pos.max()) if idx.batch else 0, total_tokens=hist_rows,
                 max_tokens=idx.max_tokens, page_size=page_size)
    return HostCase(spec=spec, index=idx, num_kv_heads=hkv, num_heads=hq, query=q, current_key=ck, current_value=cv,
                    hist_key=hk, hist_value=hv, hist_index=hist)


def cache_shapes(layout: int, max_tokens: int, num_layer: int, num_kv_heads: int, head_dim: int):
    """Shapes of (cache, scale) for a cache_layout (text_generator.cc:200-205 for layout 0)."""
    g = head_dim // 8
    if layout == 0:
        return (max_tokens, num_layer, 2, num_kv_heads, head_dim), (max_tokens, num_layer, 2, num_kv_heads, g)
    if layout == 3:
        return (num_layer, 2, num_kv_heads, max_tokens, head_dim), (num_layer, 2, num_kv_heads, max_tokens, g)
    raise ValueError("cache_layout must be 0 or 3")


def prefill_flops(num_heads: int, head_dim: int, seqlens: np.ndarray) -> float:
    """Algorithmic flops of causal prefill without history: QK^T and PV over the lower triangle
    (diagonal included), 2 * S * (S + 1) * Dh * Hq per sequence of length S."""
    s = np.asarray(seqlens, dtype=np.float64)
    return float((2.0 * s * (s + 1.0) * head_dim * num_heads).sum())


def decode_bytes(spec_heads_kv: int, head_dim: int, kvlens: np.ndarray, num_heads: int) -> int:
    """Algorithmic bytes of the decode part: cache codes + scales of every (token, kv head), K and
    V, plus the query and output rows."""
    per_tok = spec_heads_kv * 2 * (head_dim + head_dim // 8 * 2)
    return int(kvlens.sum()) * per_tok + int(kvlens.size) * 2 * num_heads * head_dim * 2


# ------------------------------------------------------------------------------------------------
# device-side builder (torch); imported lazily so that the module works without a GPU
# ------------------------------------------------------------------------------------------------

@dataclass
class DeviceCase:
    spec: Spec
    index: Index
    num_heads: int
    num_kv_heads: int
    layout: int
    num_layer: int
    layer_idx: int
    query: "object"
    current_key: "object"
    current_value: "object"
    seqstarts: "object"
    kvstarts: "object"
    cachestarts: "object"
    start_pos: "object"
    cache: "object"
    scale: "object"


class _HeadStreams:
    """One random stream per GLOBAL kv head (plus one for the token-level draws), so that the values of a
    head do not depend on how many ranks the heads are sharded over: rank r of N holds exactly the numbers
    that heads [r * Hkv / N, (r + 1) * Hkv / N) hold in the unsharded workload."""

    def __init__(self, spec: Spec, device, first_head: int, heads: int):
        import torch
        self.heads = []
        for h in range(first_head, first_head + heads):
            g = torch.Generator(device=device)
            g.manual_seed(spec.seed * 7919 + 1000 + h)
            self.heads.append(g)
        self.tokens = torch.Generator(device=device)
        self.tokens.manual_seed(spec.seed * 7919 + 999)

    def normal(self, rows, per_head, dim, device):
        """[rows, len(heads) * per_head, dim] fp32: `per_head` heads' worth of N(0,1) from every stream."""
        import torch
        out = torch.empty((rows, len(self.heads) * per_head, dim), device=device, dtype=torch.float32)
        for i, g in enumerate(self.heads):
            out[:, i * per_head:(i + 1) * per_head] = torch.randn((rows, per_head, dim), generator=g, device=device,
                                                                  dtype=torch.float32)
        return out


def _torch_kv(streams: _HeadStreams, rows, dim, spec: Spec, is_key: bool, device):
    import torch
    x = streams.normal(rows, 1, dim, device)
    if is_key and spec.outlier_k:
        x[:, :, ::16] *= 8.0
    if is_key and spec.peaked and rows > 0:
        hot = torch.rand((rows,), generator=streams.tokens, device=device) < 0.01
        x[hot] += 6.0
    return x.to(torch.float16)


def device_case(spec: Spec, device, rank: int = 0, world: int = 1, layout: int = 0, num_layer: int = 1,
                layer_idx: int = 0, slab_tokens: int = 1 << 17, page_size: int = 0) -> DeviceCase:
    """Build a workload on `device`; the cache is filled by the library's append kernel."""
    import torch
    from . import ops

    if spec.num_kv_heads % world or spec.num_heads % world:
        raise ValueError("head counts must divide by the number of ranks")
    hkv, hq, dh = spec.num_kv_heads // world, spec.num_heads // world, spec.head_dim
    idx = index_for(spec, page_size=page_size)
    gen = _HeadStreams(spec, device, rank * hkv, hkv)
    cshape, sshape = cache_shapes(layout, idx.max_tokens, num_layer, hkv, dh)
    cache = torch.zeros(cshape, dtype=torch.int8, device=device)
    scale = torch.zeros(sshape, dtype=torch.float16, device=device)

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)

    cachestarts = dev(idx.cachestarts)
    kvc = ops.KeyValueCache(ops.KeyValueCacheParam(num_layer=num_layer, layer_idx=layer_idx, quant_bit=8,
                                                   quant_group=8, cache_layout=layout,
                                                   cache_mode=1 if page_size else 0,
                                                   page_size=page_size or 128))
    lib = kvc.lib
    # history: slabs of whole sequences (long sequences are cut into several appends)
    b = 0
    B = idx.batch
    while b < B:
        # take sequences until the slab is full; a single long sequence is cut by position
        hist = int(idx.start_pos[b])
        if hist > slab_tokens:
            done = 0
            while done < hist:
                n = min(slab_tokens, hist - done)
                _append_slab(lib, kvc, spec, gen, device, hkv, dh, idx, cachestarts, cache, scale,
                             [b], [n], [done], page_size)
                done += n
            b += 1
            continue
        seqs, lens, tot = [], [], 0
        while b < B and tot + int(idx.start_pos[b]) <= slab_tokens:
            n = int(idx.start_pos[b])
            if n > 0:
                seqs.append(b)
                lens.append(n)
                tot += n
            b += 1
        if seqs:
            _append_slab(lib, kvc, spec, gen, device, hkv, dh, idx, cachestarts, cache, scale, seqs, lens,
                         [0] * len(seqs), page_size)
    T = idx.total_tokens
    q = gen.normal(T, hq // hkv, dh, device).to(torch.float16)
    ck = _torch_kv(gen, T, dh, spec, True, device)
    cv = _torch_kv(gen, T, dh, spec, False, device)
    torch.cuda.synchronize(device)
    return DeviceCase(spec=spec, index=idx, num_heads=hq, num_kv_heads=hkv, layout=layout, num_layer=num_layer,
                      layer_idx=layer_idx, query=q, current_key=ck, current_value=cv, seqstarts=dev(idx.seqstarts),
                      kvstarts=dev(idx.kvstarts), cachestarts=cachestarts, start_pos=dev(idx.start_pos), cache=cache,
                      scale=scale)


def _append_slab(lib, kvc, spec, gen, device, hkv, dh, idx, cachestarts_all, cache, scale, seqs, lens, offsets,
                 page_size):
    import torch
    from . import capi

    rows = int(sum(lens))
    hk = _torch_kv(gen, rows, dh, spec, True, device)
    hv = _torch_kv(gen, rows, dh, spec, False, device)
    seqstarts = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int64, device=device)
    start_pos = torch.tensor(offsets, dtype=torch.int64, device=device)
    sel = torch.tensor(seqs, dtype=torch.int64, device=device)
    cs = cachestarts_all.index_select(0, sel).contiguous()
    stride_b = cs.shape[1] if cs.dim() == 2 else 0
    p = kvc._params(hkv, dh, len(seqs), rows, idx.max_tokens, stride_b)
    rc = lib.kv_append(p, hk.data_ptr(), hv.data_ptr(), seqstarts.data_ptr(), cs.data_ptr(), start_pos.data_ptr(),
                       cache.data_ptr(), scale.data_ptr(), torch.cuda.current_stream().cuda_stream)
    if rc != capi.SUCCESS:
        raise RuntimeError(f"pplb200_kv_append_i8g8 failed: {lib.status_str(rc)}")
    torch.cuda.synchronize(device)  # the slab tensors are freed on return
