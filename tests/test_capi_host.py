"""Host-side checks of the C ABI that need no GPU: the library loads, exports every symbol that
include/ppl_nn_b200.h declares, validates its arguments with the reference's error codes, sizes its
workspace sensibly, and refuses to compute without an sm_100a device."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _params(lib, capi, **kw):
    p = capi.AttnParams()
    p.num_heads, p.num_kv_heads, p.head_dim, p.is_causal = 32, 8, 128, 1
    p.num_layer, p.layer_idx, p.quant_bit, p.quant_group = 1, 0, 8, 8
    p.cache_mode, p.cache_layout, p.page_size = 0, 0, 128
    p.split_k_mode = 1
    p.batch, p.decoding_batches, p.max_seqlen, p.max_kvlen = 16, 16, 1, 4096
    p.total_tokens, p.max_tokens = 16, 1 << 16
    for k, v in kw.items():
        setattr(p, k, v)
    assert lib.fill_cache_strides(p) == capi.SUCCESS or p.cache_layout not in (0, 3)
    return p


def test_header_symbols_are_all_exported(built_lib, pkg):
    from ppl_nn_b200 import capi
    header = (ROOT / "include" / "ppl_nn_b200.h").read_text()
    declared = set(re.findall(r"\b(pplb200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(capi.EXPORTS)
    for name in declared:
        assert hasattr(built_lib.dll, name), name


def test_params_struct_layout_matches_header(pkg):
    from ppl_nn_b200 import capi
    header = (ROOT / "include" / "ppl_nn_b200.h").read_text()
    body = header[header.index("typedef struct pplb200_attn_params"):header.index("} pplb200_attn_params;")]
    fields = re.findall(r"^\s*(int32_t|int64_t)\s+([a-z_]+);", body, flags=re.M)
    assert [n for _, n in fields] == [n for n, _ in capi.AttnParams._fields_]
    for (ctype, name), (_, pytype) in zip(fields, capi.AttnParams._fields_):
        assert ctypes.sizeof(pytype) == (4 if ctype == "int32_t" else 8), name
    assert ctypes.sizeof(capi.AttnParams) == 14 * 4 + 11 * 8


def test_cache_strides_follow_the_reference_layouts(built_lib, pkg):
    from ppl_nn_b200 import capi
    p = _params(built_lib, capi, num_layer=4, cache_layout=0)
    # (MaxT, L, 2, H, Dh): multi_head_cache_attention_kernel.cc:141-148
    assert (p.cache_stride_s, p.cache_stride_l, p.cache_stride_h, p.cache_stride_kv) == (4 * 2 * 8 * 128, 2 * 8 * 128,
                                                                                         128, 8 * 128)
    p = _params(built_lib, capi, num_layer=4, cache_layout=3)
    m = p.max_tokens  # (L, 2, H, MaxT, Dh): same file :149-155
    assert (p.cache_stride_s, p.cache_stride_l, p.cache_stride_h, p.cache_stride_kv) == (128, 2 * 8 * m * 128, m * 128,
                                                                                         8 * m * 128)
    p.cache_layout = 1
    assert built_lib.status_str(built_lib.fill_cache_strides(p)) == "RC_UNSUPPORTED"


@pytest.mark.parametrize("field,value,expect", [
    ("quant_bit", 4, "RC_UNSUPPORTED"),
    ("quant_group", 16, "RC_UNSUPPORTED"),
    ("head_dim", 96, "RC_UNSUPPORTED"),
    ("cache_layout", 1, "RC_UNSUPPORTED"),
    ("cache_mode", 2, "RC_UNSUPPORTED"),
    ("num_kv_heads", 5, "RC_INVALID_VALUE"),
    ("layer_idx", 3, "RC_INVALID_VALUE"),
    ("decoding_batches", 17, "RC_INVALID_VALUE"),
    ("split_k_mode", 3, "RC_INVALID_VALUE"),
    ("max_tokens", 0, "RC_INVALID_VALUE"),
])
def test_bad_attributes_are_rejected_on_the_host(built_lib, pkg, field, value, expect):
    from ppl_nn_b200 import capi
    p = _params(built_lib, capi)
    setattr(p, field, value)
    rc, _ = built_lib.mhca_workspace_size(p)
    assert built_lib.status_str(rc) == expect


def test_paged_mode_needs_2d_cachestarts(built_lib, pkg):
    from ppl_nn_b200 import capi
    p = _params(built_lib, capi, cache_mode=1, cachestart_stride_b=0)
    rc, _ = built_lib.mhca_workspace_size(p)
    assert built_lib.status_str(rc) == "RC_INVALID_VALUE"
    p.cachestart_stride_b = 64
    rc, _ = built_lib.mhca_workspace_size(p)
    assert rc == capi.SUCCESS


def test_workspace_size_grows_with_the_problem(built_lib, pkg):
    from ppl_nn_b200 import capi
    sizes = []
    for max_kvlen in (256, 4096, 65536, 1 << 20):
        rc, n = built_lib.mhca_workspace_size(_params(built_lib, capi, max_kvlen=max_kvlen))
        assert rc == capi.SUCCESS and n >= 256 and n % 256 == 0
        sizes.append(n)
    assert sizes == sorted(sizes)
    rc, off = built_lib.mhca_workspace_size(_params(built_lib, capi, max_kvlen=1 << 20, split_k_mode=0))
    assert rc == capi.SUCCESS and off <= sizes[0]  # no split, no partials
    rc, a = built_lib.mhca_workspace_size(_params(built_lib, capi, batch=64, decoding_batches=64, total_tokens=64,
                                                  max_kvlen=65536))
    assert a >= sizes[2]


def test_null_pointers_and_missing_device(built_lib, pkg):
    """Without a GPU the library must say so, not compute somewhere else."""
    import torch
    from ppl_nn_b200 import capi
    p = _params(built_lib, capi)
    fake = ctypes.c_void_p(4096)
    rc = built_lib.mhca_forward(p, None, fake, fake, fake, fake, fake, fake, fake, fake, fake, 1 << 30, fake, None)
    assert built_lib.status_str(rc) == "RC_NOT_FOUND"
    rc = built_lib.mhca_forward(p, fake, fake, fake, fake, fake, fake, fake, fake, None, fake, 1 << 30, fake, None)
    assert built_lib.status_str(rc) == "RC_UNSUPPORTED"  # scale is required: quantised cache only
    if not torch.cuda.is_available():
        assert not built_lib.device_ready()
        rc = built_lib.mhca_forward(p, fake, fake, fake, fake, fake, fake, fake, fake, fake, fake, 1 << 30, fake, None)
        assert built_lib.status_str(rc) == "RC_NO_DEVICE_CODE"
        rc = built_lib.kv_append(p, fake, fake, fake, fake, fake, fake, fake, None)
        assert built_lib.status_str(rc) == "RC_NO_DEVICE_CODE"


def test_misaligned_pointers_are_refused_before_any_launch(built_lib, pkg):
    """16-byte vector accesses and TMA on the payload tensors, 8-byte loads on the index tensors: a pointer
    that would fault on the device is an RC_INVALID_VALUE on the host."""
    from ppl_nn_b200 import capi
    p = _params(built_lib, capi)
    fake = ctypes.c_void_p(4096)
    for bad_slot, bad in ((0, 4096 + 8), (3, 4096 + 4), (7, 4096 + 2)):  # query, seqstarts, cache
        args = [fake] * 9
        args[bad_slot] = ctypes.c_void_p(bad)
        rc = built_lib.mhca_forward(p, *args, fake, 1 << 30, fake, None)
        assert built_lib.status_str(rc) == "RC_INVALID_VALUE", bad_slot
    rc = built_lib.kv_append(p, ctypes.c_void_p(4096 + 2), fake, fake, fake, fake, fake, fake, None)
    assert built_lib.status_str(rc) == "RC_INVALID_VALUE"


def test_missing_library_fails_loudly(pkg, tmp_path):
    from ppl_nn_b200 import capi
    with pytest.raises(FileNotFoundError):
        capi.Library(tmp_path / "libppl_nn_b200.so")
