"""Regenerates the golden files of this directory from the CPU oracle.

    python tests/golden/make_golden.py

The reference tree has no fixture for this path, so these are the oracle's own outputs on the tiny
configuration (seed 0), kept to pin the oracle against accidental change.  The attention output is
stored with the file-naming scheme ppl.nn's tools use for tensors, <name>-<dims>-<dtype>.dat
(tools/pplnn_llm.cc:648-700).
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
import __graft_entry__ as entry  # noqa: E402


def main():
    entry.load_package()
    from ppl_nn_b200 import workloads
    om = entry.load_oracle()
    om.build()
    orc = om.COracle()
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
    name = "attn_output-%s-fp16.dat" % "_".join(str(v) for v in out.shape)
    out.tofile(HERE / name)
    meta = {
        "config": "cfg1_tiny", "seed": 0, "kvlens": idx.kvlens.tolist(),
        "cache_sha256": hashlib.sha256(cache.tobytes()).hexdigest(),
        "scale_sha256": hashlib.sha256(scale.tobytes()).hexdigest(),
        "attn_output_file": name,
        "numpy": np.__version__,
    }
    (HERE / "cfg1_tiny.json").write_text(json.dumps(meta, indent=1) + "\n")
    print(meta)


if __name__ == "__main__":
    main()
