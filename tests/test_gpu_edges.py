"""Edge cases of the ragged batch on the GPU, against the oracle: empty sequences inside a batch, an empty
batch, a single one-token sequence, lengths beyond the max_seqlen / max_kvlen the caller announced, and index
tensors that name rows outside the cache (skipped and reported, never dereferenced)."""
import numpy as np
import pytest

from test_gpu_parity import _case_with_index, _spec, _t, run_case, torch_dev  # noqa: F401  (fixtures and helpers)

pytestmark = pytest.mark.gpu


def test_empty_prefill_sequences_inside_the_batch(orc, torch_dev, pkg):
    """seqstarts with repeated entries: sequences of zero new tokens between real ones."""
    from ppl_nn_b200 import workloads
    spec = _spec(num_heads=8, num_kv_heads=2, head_dim=128, n_decode=2, kv_dist="list", kv_list=(17, 64),
                 n_prefill=5, seed=41)
    hc = workloads.host_case(spec)
    idx = workloads.make_index([17, 64], [0, 5, 0, 130, 0])
    hc = _case_with_index(hc, idx, spec)
    run_case(orc, torch_dev, hc)


def test_single_token_single_sequence(orc, torch_dev, pkg):
    from ppl_nn_b200 import workloads
    for lens in (([1], []), ([], [1])):
        spec = _spec(num_heads=8, num_kv_heads=8, head_dim=64, n_decode=len(lens[0]), kv_dist="list",
                     kv_list=tuple(lens[0]), n_prefill=len(lens[1]), seed=42)
        hc = workloads.host_case(spec)
        hc = _case_with_index(hc, workloads.make_index(*lens), spec)
        run_case(orc, torch_dev, hc)


def test_empty_batch_is_a_no_op(torch_dev, pkg):
    import torch
    from ppl_nn_b200 import ops
    dev = torch_dev
    op = ops.MultiHeadCacheAttention(ops.MultiHeadCacheAttentionParam(num_heads=8, num_kv_heads=2, head_dim=128,
                                                                     num_layer=1, layer_idx=0, quant_bit=8))
    z = lambda *shape, dt=torch.float16: torch.zeros(shape, dtype=dt, device=dev)
    cache, scale = z(16, 1, 2, 2, 128, dt=torch.int8), z(16, 1, 2, 2, 16)
    cache.fill_(7)
    out = op.forward(z(0, 8, 128), z(0, 2, 128), z(0, 2, 128), z(1, dt=torch.int64), z(1, dt=torch.int64),
                     z(0, dt=torch.int64), z(0, dt=torch.int64), 0, 0, 0, cache, scale)
    torch.cuda.synchronize()
    assert out.shape == (0, 8, 128) and bool((cache == 7).all())


def test_lengths_beyond_the_announced_maximum_are_clamped_and_reported(orc, torch_dev, pkg, built_lib):
    """max_kvlen / max_seqlen are host scalars the caller passes; a sequence that is longer is cut there and
    the device status word says so (PPLB200_DEV_LENGTH_CLAMPED = 4), nothing is read out of bounds."""
    import torch
    from ppl_nn_b200 import ops, workloads
    dev = torch_dev
    spec = _spec(num_heads=8, num_kv_heads=2, head_dim=128, n_decode=2, kv_dist="list", kv_list=(100, 300),
                 n_prefill=1, seed=43)
    hc = workloads.host_case(spec)
    idx = workloads.make_index([100, 300], [200])
    hc = _case_with_index(hc, idx, spec)
    err, op = run_case(orc, torch_dev, hc)          # the honest call first: clean status, parity
    assert op.device_status() == 0
    Hq, Hkv, Dh = 8, 2, 128
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
    cache = torch.zeros(cshape, dtype=torch.int8, device=dev)
    scale = torch.zeros(sshape, dtype=torch.float16, device=dev)
    args = (_t(hc.query, dev), _t(hc.current_key, dev), _t(hc.current_value, dev), _t(idx.seqstarts, dev),
            _t(idx.kvstarts, dev), _t(idx.cachestarts, dev), _t(idx.start_pos, dev), idx.decoding_batches)
    out = op.forward(*args, idx.max_seqlen, 128, cache, scale)      # max_kvlen too small for the second sequence
    assert op.device_status() & 4
    assert bool(torch.isfinite(out.float()).all())
    out = op.forward(*args, 64, idx.max_kvlen, cache, scale)        # max_seqlen too small for the prefill sequence
    assert op.device_status() & 4
    assert bool(torch.isfinite(out[:idx.seqstarts[2] + 64].float()).all())


def test_rows_outside_the_cache_are_skipped_and_reported(orc, torch_dev, pkg, built_lib):
    """cachestarts / start_pos come from the caller.  A row they name outside [0, max_tokens) is neither read
    nor written; the status word carries PPLB200_DEV_ROW_OUT_OF_RANGE (8); the other sequences are served as
    usual.  Every access in these cases is guarded, so nothing can fault."""
    import torch
    from ppl_nn_b200 import ops, workloads
    dev = torch_dev
    Hq, Hkv, Dh = 8, 2, 128
    spec = _spec(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, n_decode=3, kv_dist="list", kv_list=(40, 100, 70),
                 n_prefill=1, seed=45)
    idx = workloads.make_index([40, 100, 70], [50])
    hc = _case_with_index(workloads.host_case(spec), idx, spec)
    err, op = run_case(orc, dev, hc)  # the honest call: clean status, parity
    assert op.device_status() == 0

    def history():
        cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
        cache = torch.zeros(cshape, dtype=torch.int8, device=dev)
        scale = torch.zeros(sshape, dtype=torch.float16, device=dev)
        hidx = hc.hist_index
        ops.KeyValueCache(ops.KeyValueCacheParam(num_layer=1, layer_idx=0, quant_bit=8)).forward(
            _t(hc.hist_key, dev), _t(hc.hist_value, dev), _t(hidx.seqstarts, dev), _t(hidx.kvstarts, dev),
            _t(hidx.cachestarts, dev), _t(hidx.start_pos, dev), hidx.max_seqlen, hidx.max_kvlen, cache, scale,
            total_kv=0)
        return cache, scale

    def call(cachestarts, cache, scale):
        return op.forward(_t(hc.query, dev), _t(hc.current_key, dev), _t(hc.current_value, dev),
                          _t(idx.seqstarts, dev), _t(idx.kvstarts, dev), _t(cachestarts, dev), _t(idx.start_pos, dev),
                          idx.decoding_batches, idx.max_seqlen, idx.max_kvlen, cache, scale)

    before, _ = history()
    good_cache, good_scale = history()
    good = call(idx.cachestarts, good_cache, good_scale).clone()
    assert op.device_status() == 0
    for victim, what in ((1, "beyond"), (1, "negative"), (3, "beyond")):
        cache, scale = history()
        cs = idx.cachestarts.copy()
        cs[victim] = idx.max_tokens + 5 if what == "beyond" else -7
        out = call(cs, cache, scale)
        assert op.device_status() & 8, (victim, what)
        assert bool(torch.isfinite(out.float()).all())
        # the sequences with honest indices are served as usual, bit for bit
        for b in range(idx.batch):
            if b != victim:
                lo, hi = int(idx.seqstarts[b]), int(idx.seqstarts[b + 1])
                assert bool((out[lo:hi].view(torch.int16) == good[lo:hi].view(torch.int16)).all()), (victim, what, b)
        # and the victim's new tokens were not written anywhere: its own rows still hold what they held
        expect = good_cache.clone()
        lo = int(idx.cachestarts[victim] + idx.start_pos[victim])
        hi = lo + int(idx.seqlens[victim])
        expect[lo:hi] = before[lo:hi]
        assert bool((cache == expect).all()), (victim, what)

    # paged mode: a page table too short for the announced max_kvlen is refused on the host
    pop = ops.MultiHeadCacheAttention(ops.MultiHeadCacheAttentionParam(
        num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, num_layer=1, layer_idx=0, quant_bit=8, cache_mode=1, page_size=16))
    pidx = workloads.make_index([40, 100, 70], [50], page_size=16)
    cshape, sshape = workloads.cache_shapes(0, pidx.max_tokens, 1, Hkv, Dh)
    pc, ps = torch.zeros(cshape, dtype=torch.int8, device=dev), torch.zeros(sshape, dtype=torch.float16, device=dev)
    pargs = (_t(hc.query, dev), _t(hc.current_key, dev), _t(hc.current_value, dev), _t(pidx.seqstarts, dev),
             _t(pidx.kvstarts, dev))
    with pytest.raises(ops.OpError) as ei:
        pop.forward(*pargs, _t(pidx.cachestarts[:, :3], dev), _t(pidx.start_pos, dev), pidx.decoding_batches,
                    pidx.max_seqlen, pidx.max_kvlen, pc, ps)
    assert ei.value.name == "RC_INVALID_VALUE"
    # ... and a page entry that is not a cache row is skipped and reported on the device
    table = pidx.cachestarts.copy()
    table[1, 2] = -16
    out = pop.forward(*pargs, _t(table, dev), _t(pidx.start_pos, dev), pidx.decoding_batches, pidx.max_seqlen,
                      pidx.max_kvlen, pc, ps)
    assert pop.device_status() & 8
    assert bool(torch.isfinite(out.float()).all())


def test_second_device_in_the_same_process(orc, torch_dev, pkg):
    """Per-device launch state (function attributes, device properties): a process that has used GPU 0 runs the
    same kernels on GPU 1.  Needs two GPUs."""
    import torch
    from ppl_nn_b200 import workloads
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    hc = workloads.host_case(workloads.SPECS["cfg1_tiny"])
    run_case(orc, torch.device("cuda:0"), hc)
    spec = _spec(num_heads=8, num_kv_heads=2, head_dim=128, n_decode=2, kv_dist="list", kv_list=(40, 300), n_prefill=1,
                 seed=44)
    hc2 = _case_with_index(workloads.host_case(spec), workloads.make_index([40, 300], [150]), spec)
    with torch.cuda.device(1):
        run_case(orc, torch.device("cuda:1"), hc)
        run_case(orc, torch.device("cuda:1"), hc2)
    torch.cuda.set_device(0)


def test_step_replays_from_a_cuda_graph(torch_dev, pkg):
    """The operator's launches (append, plan, decode, merge, prefill) are all stream-ordered, so a captured
    step replays with new contents in the same buffers and gives the eager result bit for bit."""
    import torch
    from ppl_nn_b200 import ops, workloads
    spec = workloads.scaled(workloads.SPECS["cfg3_llama8b_mixed"], seqs=0.125, length=0.25)
    dc = workloads.device_case(spec, torch_dev)
    idx = dc.index
    op = ops.MultiHeadCacheAttention(ops.MultiHeadCacheAttentionParam(
        num_heads=dc.num_heads, num_kv_heads=dc.num_kv_heads, head_dim=spec.head_dim, num_layer=1, layer_idx=0, quant_bit=8))
    args = (dc.query, dc.current_key, dc.current_value, dc.seqstarts, dc.kvstarts, dc.cachestarts, dc.start_pos,
            idx.decoding_batches, idx.max_seqlen, idx.max_kvlen, dc.cache, dc.scale)
    eager, replayed = torch.empty_like(dc.query), torch.empty_like(dc.query)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up off the default stream: workspace, kernel attributes, tensor maps
        op.forward(*args, attn_output=replayed)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        op.forward(*args, attn_output=replayed)
    for factor in (1.0, 0.5):
        dc.query.mul_(factor)
        op.forward(*args, attn_output=eager)
        replayed.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert op.device_status() == 0
        assert bool((eager.view(torch.int16) == replayed.view(torch.int16)).all())
