"""KV-head sharding on CPU: two gloo ranks each run the oracle on their head shard with a private
cache; the all-gathered outputs must equal the unsharded oracle output bit for bit (heads are
independent, so sharding changes no arithmetic)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_head_shard_ranges(pkg):
    from ppl_nn_b200 import sharding
    assert sharding.head_shard(64, 8, 0, 8) == (slice(0, 8), slice(0, 1))
    assert sharding.head_shard(64, 8, 7, 8) == (slice(56, 64), slice(7, 8))
    assert sharding.head_shard(32, 32, 1, 4) == (slice(8, 16), slice(8, 16))
    covered = []
    for r in range(4):
        q, kv = sharding.head_shard(32, 8, r, 4)
        covered += list(range(q.start, q.stop))
        assert (q.stop - q.start) == 4 * (kv.stop - kv.start)
    assert covered == list(range(32))
    with pytest.raises(ValueError):
        sharding.head_shard(32, 8, 0, 3)
    with pytest.raises(ValueError):
        sharding.head_shard(32, 8, 4, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    from ppl_nn_b200 import sharding, workloads
    om = entry.load_oracle()
    orc = om.COracle()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        Hq, Hkv, Dh = 8, 4, 64
        idx = workloads.make_index([17, 64, 130], [9])
        rng = np.random.default_rng(3)  # every rank draws the SAME full tensors, then keeps its shard
        T = idx.total_tokens
        q = rng.standard_normal((T, Hq, Dh), dtype=np.float32).astype(np.float16)
        ck = rng.standard_normal((T, Hkv, Dh), dtype=np.float32).astype(np.float16)
        cv = rng.standard_normal((T, Hkv, Dh), dtype=np.float32).astype(np.float16)
        rows = int(idx.start_pos.sum())
        hk = rng.standard_normal((rows, Hkv, Dh), dtype=np.float32).astype(np.float16)
        hv = rng.standard_normal((rows, Hkv, Dh), dtype=np.float32).astype(np.float16)
        hstarts = np.concatenate([[0], np.cumsum(idx.start_pos)]).astype(np.int64)
        zeros = np.zeros_like(idx.start_pos)

        def run(q_, ck_, cv_, hk_, hv_, hq, hkv):
            cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, hkv, Dh)
            cache = np.zeros(cshape, dtype=np.int8)
            scale = np.zeros(sshape, dtype=np.float16)
            kw = dict(num_heads=hq, num_kv_heads=hkv, head_dim=Dh, batch=idx.batch, max_tokens=idx.max_tokens)
            orc.kv_append(orc.desc(decoding_batches=0, **kw), hk_, hv_, hstarts, idx.cachestarts, zeros, cache, scale)
            return orc.mhca(orc.desc(decoding_batches=idx.decoding_batches, **kw), q_, ck_, cv_, idx.seqstarts,
                            idx.cachestarts, idx.start_pos, cache, scale)

        qs, kvs = sharding.head_shard(Hq, Hkv, rank, world)
        lq, lk, lv = sharding.shard_call(q, ck, cv, Hq, Hkv, rank, world)
        local = run(lq, lk, lv, np.ascontiguousarray(hk[:, kvs]), np.ascontiguousarray(hv[:, kvs]), qs.stop - qs.start,
                    kvs.stop - kvs.start)
        # gloo gathers float32 (fp16 -> fp32 is exact, so bit patterns survive the round trip)
        full = sharding.gather_heads(torch.from_numpy(local.astype(np.float32)), world)
        if rank == 0:
            want = run(q, ck, cv, hk, hv, Hq, Hkv)
            got = full.numpy().astype(np.float16)
            np.save(os.path.join(result_dir, "ok.npy"), np.array([np.array_equal(got.view(np.uint16), want.view(np.uint16))]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_result(pkg, orc, tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert bool(np.load(tmp_path / "ok.npy")[0])
