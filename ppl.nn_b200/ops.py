"""Operator-level Python face of the two ppl.nn operators, on torch CUDA tensors.

Names, attributes, input order and error behaviour follow the llm_cuda engine:
  * attributes and defaults: src/ppl/nn/models/onnx/parsers/opmx/parse_multi_head_cache_attention_param.cc:18-45,
    parse_key_value_cache_param.cc:27-48
  * input order and guards: src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/
    multi_head_cache_attention_kernel.cc:27-168 and key_value_cache_kernel.cc:26-110
torch is used for device memory and streams only; all arithmetic happens in the CUDA library.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import capi


@dataclass
class KeyValueCacheParam:
    """src/ppl/nn/params/opmx/key_value_cache_param.h:10-18 (num_layer and layer_idx are required)."""
    num_layer: int
    layer_idx: int
    quant_bit: int = 0
    quant_group: int = 8
    num_repeat: int = 1
    cache_mode: int = 0
    cache_layout: int = 0
    page_size: int = 128


@dataclass
class MultiHeadCacheAttentionParam:
    """src/ppl/nn/params/opmx/multi_head_cache_attention_param.h:10-22."""
    num_heads: int
    head_dim: int
    num_layer: int
    layer_idx: int
    num_kv_heads: int = -1  # parser default: num_heads
    is_causal: bool = True
    is_alibi: bool = False
    quant_bit: int = 0
    quant_group: int = 8
    cache_mode: int = 0
    cache_layout: int = 0
    page_size: int = 128

    def __post_init__(self):
        if self.num_kv_heads < 0:
            self.num_kv_heads = self.num_heads


@dataclass
class MultiHeadAttentionParam:
    """src/ppl/nn/params/opmx/multi_head_attention_param.h."""
    num_heads: int
    head_dim: int
    num_kv_heads: int = -1  # parser default: num_heads
    is_causal: bool = True
    is_alibi: bool = False

    def __post_init__(self):
        if self.num_kv_heads < 0:
            self.num_kv_heads = self.num_heads


@dataclass
class RotaryPositionEmbeddingParam:
    """src/ppl/nn/params/opmx/rotary_position_embedding_param.h; scaling_type "" | "linear" | "dynamic"."""
    theta: float = 10000.0
    bypass_key: int = 0
    rotary_dim: int = 0
    max_position_embeddings: int = 2048
    scaling_type: str = ""
    scaling_factor: float = 1.0


@dataclass
class EngineConfig:
    """The knobs of src/ppl/nn/engines/llm_cuda/engine_config.h:30-35 that reach this path."""
    enable_cache_prefill: bool = False
    specify_decoding_attn_split_k: int = 1
    # accepted for compatibility, ignored: there is one decode algorithm here
    enable_decoding_sharemem_mhca: bool = True
    enable_decoding_infinity_mhca: bool = True
    enable_decoding_infinity_gqca: bool = True
    specify_decoding_attn_tpb: int = 0


class OpError(RuntimeError):
    """An operator returned a non-success RetCode; ``name`` is the RetCode's name."""

    def __init__(self, name: str, msg: str):
        super().__init__(f"{name}: {msg}")
        self.name = name


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(**tensors):
    for name, t in tensors.items():
        if t is None:
            raise OpError("RC_NOT_FOUND", f'Input "{name}" is required.')
        if not t.is_cuda:
            raise OpError("RC_INVALID_VALUE", f"{name} must be a CUDA tensor")
        if not t.is_contiguous():
            raise OpError("RC_INVALID_VALUE", f"{name} must be contiguous")


def _mask_arg(attn_mask):
    """The optional attn_mask input as the C ABI wants it; a tensor of zero elements is "absent", as in the
    reference (multi_head_cache_attention_kernel.cc:107)."""
    if attn_mask is None or attn_mask.numel() == 0:
        return None
    _require_cuda(attn_mask=attn_mask)
    if attn_mask.dtype != torch.float16:
        raise OpError("RC_UNSUPPORTED", "attn_mask must be fp16")
    if attn_mask.dim() not in (2, 3):
        raise OpError("RC_INVALID_VALUE", "attn_mask must be [T, C] or [num_heads, T, C]")
    return capi.AttnMask.of(attn_mask.data_ptr(), tuple(attn_mask.shape))


def _max_tokens(cache: torch.Tensor, layout: int) -> int:
    if layout == 0:
        return cache.shape[0]
    if layout == 3:
        return cache.shape[3]
    raise OpError("RC_UNSUPPORTED", "currently only support cache_layout == 0 or cache_layout == 3")


class _Base:
    def __init__(self):
        self.lib = capi.library()

    def _raise(self, fn: str, rc: int):
        if rc != capi.SUCCESS:
            raise OpError(self.lib.status_str(rc), f"{fn} failed")


class MultiHeadCacheAttention(_Base):
    """opmx.dynamic_batching.MultiHeadCacheAttention."""

    def __init__(self, param: MultiHeadCacheAttentionParam, config: EngineConfig | None = None):
        super().__init__()
        self.param = param
        self.config = config or EngineConfig()
        self._workspace: torch.Tensor | None = None

    def make_params(self, *, batch, decoding_batches, max_seqlen, max_kvlen, total_tokens, max_tokens,
                    cachestart_stride_b=0, phase_mask=0) -> capi.AttnParams:
        a, c = self.param, self.config
        p = capi.AttnParams()
        p.num_heads, p.num_kv_heads, p.head_dim = a.num_heads, a.num_kv_heads, a.head_dim
        p.is_causal = int(a.is_causal)
        p.num_layer, p.layer_idx = a.num_layer, a.layer_idx
        p.quant_bit, p.quant_group = a.quant_bit, a.quant_group
        p.cache_mode, p.cache_layout, p.page_size = a.cache_mode, a.cache_layout, a.page_size
        p.enable_cache_prefill = int(c.enable_cache_prefill)
        p.split_k_mode = int(c.specify_decoding_attn_split_k)
        p.phase_mask = phase_mask
        p.batch, p.decoding_batches = batch, decoding_batches
        p.max_seqlen, p.max_kvlen = max_seqlen, max_kvlen
        p.total_tokens, p.max_tokens = total_tokens, max_tokens
        p.cachestart_stride_b = cachestart_stride_b
        self._raise("pplb200_fill_cache_strides", self.lib.fill_cache_strides(p))
        return p

    def workspace_for(self, p: capi.AttnParams, device) -> torch.Tensor:
        rc, nbytes = self.lib.mhca_workspace_size(p)
        self._raise("pplb200_mhca_workspace_size", rc)
        if self._workspace is None or self._workspace.numel() < nbytes or self._workspace.device != device:
            # grow-only scratch, like the engine's tmp-buffer pool (llm_cuda_device.h:151-156)
            self._workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        return self._workspace

    def forward(self, query, current_key, current_value, seqstarts, kvstarts, cachestarts, start_pos,
                decoding_batches: int, max_seqlen: int, max_kvlen: int, cache, scale=None, attn_mask=None,
                attn_output: torch.Tensor | None = None, phase_mask: int = 0) -> torch.Tensor:
        a = self.param
        _require_cuda(query=query, current_key=current_key, current_value=current_value, seqstarts=seqstarts,
                      kvstarts=kvstarts, cachestarts=cachestarts, start_pos=start_pos, cache=cache)
        if a.is_alibi:
            raise OpError("RC_UNSUPPORTED", "currently only support is_alibi == false")
        if scale is None or scale.numel() == 0:
            raise OpError("RC_UNSUPPORTED", "currently only support qunatized cache but scale not found")
        mask = _mask_arg(attn_mask)
        _require_cuda(scale=scale)
        stride_b = 0
        if a.cache_mode == 1:
            if cachestarts.dim() != 2:
                raise OpError("RC_INVALID_VALUE", "cachestarts must be a 2d tensor in cache_mode 1")
            stride_b = cachestarts.shape[1]
        batch = start_pos.shape[0]
        p = self.make_params(batch=batch, decoding_batches=int(decoding_batches), max_seqlen=int(max_seqlen),
                             max_kvlen=int(max_kvlen), total_tokens=query.shape[0],
                             max_tokens=_max_tokens(cache, a.cache_layout), cachestart_stride_b=stride_b,
                             phase_mask=phase_mask)
        if attn_output is None:
            attn_output = torch.empty_like(query)
        ws = self.workspace_for(p, query.device)
        if mask is None:
            rc = self.lib.mhca_forward(p, _ptr(query), _ptr(current_key), _ptr(current_value), _ptr(seqstarts),
                                       _ptr(kvstarts), _ptr(cachestarts), _ptr(start_pos), _ptr(cache), _ptr(scale),
                                       _ptr(ws), ws.numel(), _ptr(attn_output), _stream())
        else:
            rc = self.lib.mhca_forward_masked(p, _ptr(query), _ptr(current_key), _ptr(current_value), _ptr(seqstarts),
                                              _ptr(kvstarts), _ptr(cachestarts), _ptr(start_pos), _ptr(cache),
                                              _ptr(scale), mask, _ptr(ws), ws.numel(), _ptr(attn_output), _stream())
        self._raise("pplb200_mhca_forward", rc)
        self._last_params = p
        return attn_output

    def device_status(self) -> int:
        """Status word left by the kernels of the last forward (synchronises the stream)."""
        if self._workspace is None:
            return 0
        rc, s = self.lib.mhca_device_status(_ptr(self._workspace), _stream())
        self._raise("pplb200_mhca_device_status", rc)
        return s


class KeyValueCache(_Base):
    """opmx.dynamic_batching.KeyValueCache: append, then return the dequantised history."""

    def __init__(self, param: KeyValueCacheParam):
        super().__init__()
        self.param = param

    def _params(self, num_kv_heads, head_dim, batch, total_tokens, max_tokens, stride_b) -> capi.AttnParams:
        a = self.param
        p = capi.AttnParams()
        p.num_heads = p.num_kv_heads = num_kv_heads
        p.head_dim = head_dim
        p.is_causal = 1
        p.num_layer, p.layer_idx = a.num_layer, a.layer_idx
        p.quant_bit, p.quant_group = a.quant_bit, a.quant_group
        p.cache_mode, p.cache_layout, p.page_size = a.cache_mode, a.cache_layout, a.page_size
        p.batch, p.total_tokens, p.max_tokens = batch, total_tokens, max_tokens
        p.cachestart_stride_b = stride_b
        self._raise("pplb200_fill_cache_strides", self.lib.fill_cache_strides(p))
        return p

    def forward(self, current_key, current_value, seqstarts, kvstarts, cachestarts, start_pos, max_seqlen: int,
                max_kvlen: int, cache, scale=None, total_kv: int | None = None):
        a = self.param
        _require_cuda(current_key=current_key, current_value=current_value, seqstarts=seqstarts, kvstarts=kvstarts,
                      cachestarts=cachestarts, start_pos=start_pos, cache=cache)
        if scale is None:
            raise OpError("RC_UNSUPPORTED", "currently only support qunatized cache but scale not found")
        if a.num_repeat != 1:
            raise OpError("RC_UNSUPPORTED", "currently only support num_repeat == 1")
        if current_key.dtype != torch.float16:
            raise OpError("RC_UNSUPPORTED", "currently only support fp16")
        _require_cuda(scale=scale)
        stride_b = cachestarts.shape[1] if (a.cache_mode == 1 and cachestarts.dim() == 2) else 0
        if a.cache_mode == 1 and cachestarts.dim() != 2:
            raise OpError("RC_INVALID_VALUE", "cachestarts must be a 2d tensor in cache_mode 1")
        T, Hkv, Dh = current_key.shape
        batch = start_pos.shape[0]
        p = self._params(Hkv, Dh, batch, T, _max_tokens(cache, a.cache_layout), stride_b)
        s = _stream()
        self._raise("pplb200_kv_append_i8g8",
                    self.lib.kv_append(p, _ptr(current_key), _ptr(current_value), _ptr(seqstarts), _ptr(cachestarts),
                                       _ptr(start_pos), _ptr(cache), _ptr(scale), s))
        if total_kv is None:
            # shape inference reads kvstarts[-1] on the host, as the reference op does
            # (ops/opmx/dynamic_batching/key_value_cache_op.cc:37-56)
            total_kv = int(kvstarts[-1].item())
        key = torch.empty((total_kv, Hkv, Dh), dtype=torch.float16, device=current_key.device)
        value = torch.empty_like(key)
        self._raise("pplb200_kv_gather_dequant",
                    self.lib.kv_gather_dequant(p, _ptr(kvstarts), _ptr(cachestarts), _ptr(cache), _ptr(scale),
                                               total_kv, _ptr(key), _ptr(value), s))
        return key, value


class MultiHeadAttention(_Base):
    """opmx.dynamic_batching.MultiHeadAttention: attention over this call's own key/value tensors, no cache
    (src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/multi_head_attention_kernel.cc:24-128)."""

    def __init__(self, param: MultiHeadAttentionParam):
        super().__init__()
        self.param = param
        self._workspace: torch.Tensor | None = None

    def forward(self, query, key, value, seqstarts, kvstarts, decoding_batches: int, max_seqlen: int, max_kvlen: int,
                attn_mask=None, attn_output: torch.Tensor | None = None) -> torch.Tensor:
        a = self.param
        _require_cuda(query=query, key=key, value=value, seqstarts=seqstarts, kvstarts=kvstarts)
        if a.is_alibi:
            raise OpError("RC_UNSUPPORTED", "currently only support is_alibi == false")
        mask = _mask_arg(attn_mask)
        p = capi.MhaParams()
        p.num_heads, p.num_kv_heads, p.head_dim, p.is_causal = a.num_heads, a.num_kv_heads, a.head_dim, int(a.is_causal)
        p.batch = seqstarts.shape[0] - 1
        p.decoding_batches = int(decoding_batches)
        p.max_seqlen, p.max_kvlen = int(max_seqlen), int(max_kvlen)
        p.total_tokens, p.total_kv_tokens = query.shape[0], key.shape[0]
        if attn_output is None:
            attn_output = torch.empty_like(query)
        if self._workspace is None or self._workspace.device != query.device:
            self._workspace = torch.empty(256, dtype=torch.uint8, device=query.device)
        rc = self.lib.mha_forward_masked(p, _ptr(query), _ptr(key), _ptr(value), _ptr(seqstarts), _ptr(kvstarts), mask,
                                         _ptr(self._workspace), self._workspace.numel(), _ptr(attn_output), _stream())
        self._raise("pplb200_mha_forward", rc)
        return attn_output

    def device_status(self) -> int:
        if self._workspace is None:
            return 0
        rc, status = self.lib.mhca_device_status(_ptr(self._workspace), _stream())
        self._raise("pplb200_mhca_device_status", rc)
        return status


class RotaryPositionEmbedding(_Base):
    """opmx.dynamic_batching.RotaryPositionEmbedding
    (src/ppl/nn/engines/llm_cuda/kernels/opmx/dynamic_batching/rotary_position_embedding_kernel.cc:24-132),
    and ``forward_fused``: the same rotation fused with the quantise-and-append of the KV cache."""

    _SCALING = {"": 0, "linear": 1, "dynamic": 2}

    def __init__(self, param: RotaryPositionEmbeddingParam):
        super().__init__()
        if param.scaling_type not in self._SCALING:
            raise OpError("RC_UNSUPPORTED", f"unsupported scaling_type: {param.scaling_type}")
        self.param = param
        self._workspace: torch.Tensor | None = None

    def _params(self, query, key, start_pos, max_seqlen) -> capi.RopeParams:
        a = self.param
        p = capi.RopeParams()
        p.num_heads, p.num_kv_heads, p.head_dim = query.shape[1], key.shape[1], query.shape[2]
        p.rotary_dim, p.bypass_key = a.rotary_dim, int(a.bypass_key)
        p.scaling_type = self._SCALING[a.scaling_type]
        p.max_position_embeddings = a.max_position_embeddings
        p.theta, p.scaling_factor = a.theta, a.scaling_factor
        p.batch, p.max_seqlen, p.total_tokens = start_pos.shape[0], int(max_seqlen), query.shape[0]
        return p

    def _ws(self, p, device) -> torch.Tensor:
        rc, nbytes = self.lib.rope_workspace_size(p)
        self._raise("pplb200_rope_workspace_size", rc)
        if self._workspace is None or self._workspace.numel() < nbytes or self._workspace.device != device:
            self._workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        return self._workspace

    def forward(self, query, key, seqstarts, start_pos, max_seqlen: int, rotated_query=None, rotated_key=None):
        _require_cuda(query=query, key=key, seqstarts=seqstarts, start_pos=start_pos)
        if query.dtype != torch.float16:
            raise OpError("RC_UNSUPPORTED", "currently only support fp16")
        p = self._params(query, key, start_pos, max_seqlen)
        ws = self._ws(p, query.device)
        rotated_query = torch.empty_like(query) if rotated_query is None else rotated_query
        rotated_key = torch.empty_like(key) if rotated_key is None else rotated_key
        rc = self.lib.rope_forward(p, _ptr(query), _ptr(key), _ptr(seqstarts), _ptr(start_pos), _ptr(ws), ws.numel(),
                                   _ptr(rotated_query), _ptr(rotated_key), _stream())
        self._raise("pplb200_rope_forward", rc)
        return rotated_query, rotated_key

    def forward_fused(self, attn: "MultiHeadCacheAttention", query, key, value, seqstarts, cachestarts, start_pos,
                      max_seqlen: int, cache, scale, want_rotated_key: bool = True):
        """Rotate, then quantise-and-append in the same kernel.  Returns (rotated_query, rotated_key or None);
        follow with ``attn.forward(..., phase_mask=PHASE_DECODE | PHASE_PREFILL)``."""
        _require_cuda(query=query, key=key, value=value, seqstarts=seqstarts, cachestarts=cachestarts,
                      start_pos=start_pos, cache=cache, scale=scale)
        p = self._params(query, key, start_pos, max_seqlen)
        ws = self._ws(p, query.device)
        ap = attn.make_params(batch=start_pos.shape[0], decoding_batches=0, max_seqlen=int(max_seqlen),
                              max_kvlen=0, total_tokens=query.shape[0],
                              max_tokens=_max_tokens(cache, attn.param.cache_layout),
                              cachestart_stride_b=cachestarts.shape[1] if cachestarts.dim() == 2 else 0)
        rotated_query = torch.empty_like(query)
        rotated_key = torch.empty_like(key) if want_rotated_key else None
        rc = self.lib.rope_kv_append(p, ap, _ptr(query), _ptr(key), _ptr(value), _ptr(seqstarts), _ptr(cachestarts),
                                     _ptr(start_pos), _ptr(ws), ws.numel(), _ptr(rotated_query), _ptr(rotated_key),
                                     _ptr(cache), _ptr(scale), _stream())
        self._raise("pplb200_rope_kv_append_i8g8", rc)
        return rotated_query, rotated_key
