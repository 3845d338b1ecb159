"""The step driver (ppl.nn_b200/generation.py) against the semantics of
tools/benchmark_llama/generation_state.cc, and a multi-step generation on the GPU against the oracle:
the cache is state that every step appends to, so its content after N steps, and every step's output,
must match a CPU run of the same steps."""
import numpy as np
import pytest


def _requests(pkg):
    from ppl_nn_b200.generation import Request
    return [Request(5, 3), Request(2, 1), Request(9, 4), Request(1, 2)]


@pytest.mark.parametrize("mode", [0, 1])
def test_index_semantics(pkg, mode):
    from ppl_nn_b200.generation import GenerationState
    st = GenerationState(cache_mode=mode, page_size=4)
    st.prepare(_requests(pkg))
    assert st.max_steps == 4 and st.total_input_length == 17 and st.total_output_length == 10
    if mode == 0:
        assert st.total_cache_length == 7 + 2 + 12 + 2
    else:
        assert st.total_cache_pages == 2 + 1 + 3 + 1 and st.max_cache_pages == 3
    ios = list(st.steps())
    assert len(ios) == 4
    a = ios[0]  # all prefill
    assert a.decoding_batches == 0 and a.seq_starts.tolist() == [0, 5, 7, 16, 17] and a.kv_starts.tolist() == [0, 5, 7, 16, 17]
    assert a.start_pos.tolist() == [0, 0, 0, 0] and a.max_seq_len == 9 and a.max_kv_len == 9
    if mode == 0:
        assert a.cache_indices.tolist() == [0, 7, 9, 21]
    else:
        assert a.cache_indices.tolist() == [[0, 4, 0], [8, 0, 0], [12, 16, 20], [24, 0, 0]]
    b = ios[1]  # request 1 (generation_len 1) has left
    assert b.batch_slots.tolist() == [0, 2, 3] and b.decoding_batches == 3
    assert b.start_pos.tolist() == [5, 9, 1] and b.kv_lengths.tolist() == [6, 10, 2] and b.seq_starts.tolist() == [0, 1, 2, 3]
    assert b.max_seq_len == 1 and b.max_kv_len == 10
    if mode == 0:
        assert b.cache_indices.tolist() == [0, 9, 21]
    c = ios[2]  # request 3 (generation_len 2) has left
    assert c.batch_slots.tolist() == [0, 2] and c.start_pos.tolist() == [6, 10]
    d = ios[3]
    assert d.batch_slots.tolist() == [2] and d.start_pos.tolist() == [11] and d.max_kv_len == 12
    with pytest.raises(ValueError):
        from ppl_nn_b200.generation import Request
        st.prepare([Request(3, 0)])


@pytest.mark.gpu
@pytest.mark.parametrize("mode,layout", [(0, 0), (0, 3), (1, 0)])
def test_multi_step_generation_matches_oracle(pkg, orc, built_lib, mode, layout):
    import torch
    from ppl_nn_b200 import ops, workloads
    from ppl_nn_b200.generation import GenerationState, Request
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    Hq, Hkv, Dh, page = 8, 2, 128, 16
    rng = np.random.default_rng(21)
    reqs = [Request(int(p), int(g)) for p, g in zip(rng.integers(1, 200, 6), rng.integers(1, 7, 6))]
    st = GenerationState(cache_mode=mode, page_size=page)
    st.prepare(reqs)
    max_tokens = st.total_cache_length
    cshape, sshape = workloads.cache_shapes(layout, max_tokens, 1, Hkv, Dh)
    cache_h, scale_h = np.zeros(cshape, dtype=np.int8), np.zeros(sshape, dtype=np.float16)
    cache_d, scale_d = torch.zeros(cshape, dtype=torch.int8, device=dev), torch.zeros(sshape, dtype=torch.float16, device=dev)
    op = ops.MultiHeadCacheAttention(ops.MultiHeadCacheAttentionParam(
        num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, num_layer=1, layer_idx=0, quant_bit=8, cache_mode=mode,
        cache_layout=layout, page_size=page))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    worst = 0.0
    for step, io in enumerate(st.steps()):
        T = int(io.seq_starts[-1])
        q = rng.standard_normal((T, Hq, Dh)).astype(np.float16)
        k = rng.standard_normal((T, Hkv, Dh)).astype(np.float16)
        v = rng.standard_normal((T, Hkv, Dh)).astype(np.float16)
        d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=io.batch, decoding_batches=io.decoding_batches,
                     max_tokens=max_tokens, cache_mode=mode, cache_layout=layout, page_size=page,
                     cachestart_stride_b=io.cache_indices.shape[1] if mode == 1 else 0)
        want = orc.mhca(d, q, k, v, io.seq_starts, io.cache_indices, io.start_pos, cache_h, scale_h).astype(np.float32)
        got = op.forward(t(q), t(k), t(v), t(io.seq_starts), t(io.kv_starts), t(io.cache_indices), t(io.start_pos),
                         io.decoding_batches, io.max_seq_len, io.max_kv_len, cache_d, scale_d)
        assert op.device_status() == 0
        err = np.abs(got.cpu().numpy().astype(np.float32) - want)
        assert err.max() <= 2e-3 and err.mean() <= 1e-3, (step, err.max(), err.mean())
        worst = max(worst, float(err.max()))
        # the cache is state: after every step both copies hold the same codes and scales
        np.testing.assert_array_equal(cache_d.cpu().numpy(), cache_h)
        np.testing.assert_array_equal(scale_d.cpu().numpy().view(np.uint16), scale_h.view(np.uint16))
    print(f"[parity] generation mode {mode} layout {layout}: {st.max_steps} steps, worst max-abs {worst:.3e}")
