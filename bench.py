#!/usr/bin/env python
"""Benchmark of the INT8-KV cache attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One *step* is one call of the MultiHeadCacheAttention operator (quantise-and-append of the new
token of every sequence, then ragged split-k decode attention over the INT8 cache) on one
transformer layer.  The headline workload is the LLaMA-2-7B pure-decode configuration: 256
sequences, MHA 32 heads x 128, KV lengths uniform in [128, 4096], seed 1, N(0,1) values with
every 16th K channel scaled by 8; the cache is 5.6 GB, far larger than the 126 MB L2, so no
flush is needed between steps.  With N > 1 the KV heads (and their query heads) are sharded over
the ranks exactly like tensor parallelism shards them; there is no collective in the timed path,
total work is fixed, so the run is a strong-scaling run.  After timing, the shards' outputs are
gathered with NCCL and two kv heads are recomputed on rank 0 from scratch as a one-head workload
(head values do not depend on the sharding) and compared with the gathered columns.

Rank 0 prints ONE JSON line.
  value       decode tokens per second of the whole job with all inputs resident in HBM, from exactly
              --steps timed steps after --warmup warm-up steps;
  sustained   the same loop repeated until the timed region is at least half a second long
              (a 20-step region lasts 18 ms, too short to see the clocks settle under the power cap);
  e2e         the same metric through the reference-facing operator (the C++ Op/Kernel classes of
              ppl.nn_b200/host, created via the registry) with HOST inputs: pinned host -> device copies of
              query/key/value and the index tensors and a device -> host copy of the attention output,
              every step, inside the timed region (the KV cache itself is device-resident state by the
              operator's contract);
  roofline    the dominant kernel (decode_splitk_kernel), timed with CUDA events on its own stream
              inside the library during the timed steps;
  per_config  the other benchmark configurations in the same invocation (mixed continuous-batching step
              with its tcgen05 prefill kernel, the same with prefill from the INT8 cache, the 70B-shape
              large-batch decode, the long-context step), each sharded over the same N ranks;
  cpu_baseline  the CPU restatement of the graph the reference's x86 engine would run for this
              mathematics (oracle/x86_graph_baseline.c, OpenMP over all host threads) on a bounded
              sample of the headline workload.

`--impl reference` times that CPU restatement alone (the reference's CUDA kernels are not part
of its source tree and nothing of it builds here).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

METRIC = "ragged INT8-KV decode attn: HBM GB/s (% of peak) and tokens/s at 1/2/4/8 B200"
DEFAULT_WORKLOAD = "cfg2_llama7b_decode"
FALLBACK_HBM_GBS = 6650.0
DTYPE = "fp16 in/out, int8 cache, fp32 accumulate"

# DRAM bytes moved by decode_splitk_kernel per algorithmic byte, from an ncu capture of one launch on one
# eighth of the headline workload (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes
# of the captured launch: 693.08 MB + 4.61 MB for 690.86 MB); traffic grows in proportion to cached tokens.
DECODE_TRAFFIC_PER_ALGO_BYTE = 1.0099

def decode_scores_form(spec) -> str:
    """Which form of the decode kernel the library picks for a workload (csrc/decode_splitk.cu, launch_decode_dh)."""
    if spec.n_decode == 0:
        return "none (no decode sequences)"
    if spec.num_heads == spec.num_kv_heads and os.environ.get("PPLB200_DECODE_KDOT", "1")[:1] != "0":
        return "integer dot products (one query head per kv head)"
    return "tensor cores (mma.m16n8k16 over the dequantised keys)"


PER_CONFIG = (  # (workload, enable_cache_prefill)
    ("cfg3_llama8b_mixed", False),
    ("cfg3_llama8b_mixed", True),
    ("cfg4_llama70b_decode", False),
    ("cfg5_longctx", False),
)


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]),
                    "tflops_sustained": float(d["bf16_tflops_sustained"]),
                    "source": "measured on this machine pool (copy read+write bandwidth; cuBLAS bf16 burst / sustained)"}
        except Exception:
            pass
    return {"hbm_gbs": FALLBACK_HBM_GBS, "tflops": 1590.0, "tflops_sustained": 1400.0,
            "source": "fallback (6.65 TB/s, 1.59 / 1.4 PFLOP/s: an earlier measurement on the same kind of machine)"}


# ------------------------------------------------------------------------------------------------
# clocks: NVML samples taken while the timed regions run (read-only)
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, device_index: int, period_s: float = 0.001):
        self.rows = []  # (perf_counter, sm_mhz, mem_mhz, watts, reason mask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            import torch
            props = torch.cuda.get_device_properties(device_index)
            bus = props.pci_bus_id if hasattr(props, "pci_bus_id") else None
            self._h = None
            if bus is not None:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    if pynvml.nvmlDeviceGetPciInfo(h).bus == bus:
                        self._h = h
                        break
            if self._h is None:
                vis = os.environ.get("CUDA_VISIBLE_DEVICES")
                phys = int(vis.split(",")[device_index]) if vis and vis.split(",")[device_index].isdigit() \
                    else device_index
                self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # no NVML: report that instead of inventing clocks
            self._nv, self._h = None, None
            self.error = repr(exc)

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.rows.append((time.perf_counter(),
                                  int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)),
                                  int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_MEM)),
                                  nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0,
                                  int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))))
            except Exception:
                pass
            self._stop.wait(self._period)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self, t0: float | None = None, t1: float | None = None):
        """Clocks between two perf_counter stamps (the whole sampling period without them)."""
        if self._h is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": getattr(self, "error", "no NVML")}
        rows = [r for r in self.rows if (t0 is None or r[0] >= t0) and (t1 is None or r[0] <= t1)]
        reasons = set()
        for r in rows:
            for bit, name in self.REASONS.items():
                if r[4] & bit and name != "gpu_idle":
                    reasons.add(name)
        sm = [r[1] for r in rows]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons), "samples": len(rows),
                "mem_mhz": int(statistics.median([r[2] for r in rows])) if rows else None,
                "power_w_max": round(max(r[3] for r in rows), 1) if rows else None}


# ------------------------------------------------------------------------------------------------
# CPU arm: the x86-graph restatement on the host cores
# ------------------------------------------------------------------------------------------------
def _load_x86_baseline():
    import importlib.util
    name = "x86_graph_baseline"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, ROOT / "oracle" / "x86_graph_baseline.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def cpu_time_sample(spec, num_seqs: int, target_seconds: float = 12.0, steps: int | None = None, warmup: int = 1):
    """Time the CPU restatement of the x86 graph on the first `num_seqs` decode sequences of `spec` (same
    seeded lengths; random valid codes and scales: the arithmetic does not depend on them).  The cache is
    dequantised to fp32 BEFORE the timed region, as the graph runs over the dequantised cache; a second figure
    includes one dequantisation per step.  With `steps` the run is exactly `warmup` + `steps` passes, otherwise
    as many passes as fill `target_seconds`.  Returns a dict."""
    from ppl_nn_b200 import workloads
    xb = _load_x86_baseline()
    base = xb.X86GraphBaseline(native=True)
    kv_all, _ = workloads.draw_lengths(spec)
    Hq, Hkv, Dh = spec.num_heads, spec.num_kv_heads, spec.head_dim
    # bound the dequantised sample (fp32 K and V) to about 3 GB of host memory
    per_seq = float(kv_all.mean()) * Hkv * Dh * 8
    num_seqs = int(max(1, min(num_seqs, spec.n_decode, 3.0e9 // per_seq)))
    kv = kv_all[:num_seqs]
    rng = np.random.default_rng(99)
    idx = workloads.make_index(kv, [])
    cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
    cache = rng.integers(-127, 128, size=cshape, dtype=np.int8)
    scale = rng.uniform(0.01, 0.05, size=sshape).astype(np.float16)
    q = rng.standard_normal((num_seqs, Hq, Dh), dtype=np.float32).astype(np.float16)
    st = base.prepare(Hkv, Dh, kv, idx.cachestarts, cache, scale)
    out = np.empty((num_seqs, Hq, Dh), dtype=np.float16)
    base.dequant(st)  # first touch of the fp32 matrices
    t0 = time.perf_counter()
    base.dequant(st)
    dequant_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    base.attention(st, q, out)
    one = time.perf_counter() - t0
    if steps is None:
        steps = max(3, min(500, int(target_seconds / max(one, 1e-5))))
    for _ in range(max(warmup - 1, 0)):
        base.attention(st, q, out)
    t0 = time.perf_counter()
    for _ in range(steps):
        base.attention(st, q, out)
    per_step = (time.perf_counter() - t0) / steps
    cores = base.num_threads()
    sample = (f"first {num_seqs} of {spec.n_decode} sequences of {spec.name} (same seeded KV lengths, "
              f"{int(kv.sum())} cached tokens), per (sequence, head) fp32 GEMV -> scale -> softmax -> GEMV over the "
              f"dequantised cache, {steps} passes, OpenMP x{cores}, gcc -O3 -march=native")
    return {"value": num_seqs / per_step, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
            "ms_per_step_of_sample": per_step * 1e3, "steps": steps,
            "value_including_dequantisation": num_seqs / (per_step + dequant_s),
            "dequantisation_ms_of_sample": dequant_s * 1e3,
            "fp32_gbs": float(kv.sum()) * Hkv * Dh * 8 / per_step / 1e9}


def run_reference_arm(args, rank: int):
    """`--impl reference`: the reference's CUDA kernels are absent from its tree and nothing of it
    compiles here, so this arm is the CPU restatement of the graph its x86 engine would run, on all host
    threads.  One step = one pass over the bounded sample; exactly K steps after W warm-ups."""
    if rank != 0:
        return
    entry.load_package()
    from ppl_nn_b200 import workloads
    spec = workloads.SPECS[args.workload]
    cpu = cpu_time_sample(spec, args.cpu_seqs, steps=args.steps, warmup=max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": cpu["steps"], "warmup": max(args.warmup, 1), "ms_per_step": cpu["ms_per_step_of_sample"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": spec.name, "sample": cpu["sample"]},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the per-sequence MatMul/Softmax/MatMul graph of the reference's x86 engine "
                "(oracle/x86_graph_baseline.c); the reference's own kernels for this path live in the un-vendored "
                "ppl.llm.kernel.cuda and ppl.kernel.cpu and do not exist in its tree",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class Ctx:
    """What every workload run needs: device, ranks, the library, the roofline denominators."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {self.world}: launch with torch.distributed.run")
        entry.load_package()
        from ppl_nn_b200 import capi
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
        self.dev = torch.device("cuda", self.local_rank)
        torch.cuda.set_device(self.dev)
        self.lib = capi.library()
        if not self.lib.device_ready():
            raise SystemExit("the CUDA library has no sm_100a code for this device")
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = _peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, values):
        if self.world == 1:
            return [float(v) for v in values]
        t = self.torch.tensor(list(values), device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]


def make_op(dc, spec, layout, page_size, cache_prefill=False):
    from ppl_nn_b200 import ops
    paging = dict(cache_mode=1, page_size=page_size) if page_size else {}
    return ops.MultiHeadCacheAttention(
        ops.MultiHeadCacheAttentionParam(num_heads=dc.num_heads, num_kv_heads=dc.num_kv_heads, head_dim=spec.head_dim,
                                         num_layer=1, layer_idx=0, quant_bit=8, cache_layout=layout, **paging),
        ops.EngineConfig(enable_cache_prefill=cache_prefill))


def timed_steps(ctx: Ctx, step, steps: int, warmup: int, min_seconds: float = 0.0):
    """W warm-up steps, then exactly `steps` timed steps between barriers, CUDA events on the launching
    stream, max over ranks.  Every fourth timed step has its kernels bracketed by the library's own event
    pairs (four event records cost a few microseconds, which shows on a 150 us step of an 8-way shard); the
    others run exactly as a caller would run them.  With `min_seconds` the same K-step block is repeated
    until that much time has been timed ("sustained").  Returns a dict of times."""
    from ppl_nn_b200 import capi
    torch, lib = ctx.torch, ctx.lib
    for _ in range(warmup):
        step()
    ctx.barrier()
    for fam in (capi.KERNEL_DECODE, capi.KERNEL_APPEND, capi.KERNEL_PREFILL):
        lib.profile_read(fam)
    launches0 = lib.launch_count()
    blocks = []  # ms of each K-step block (max over ranks)
    stamps = []
    total_ms = 0.0
    while True:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        w0 = time.perf_counter()
        e0.record()
        for i in range(steps):
            lib.profile_enable(i % 4 == 0)
            step()
        e1.record()
        ctx.barrier()
        w1 = time.perf_counter()
        lib.profile_enable(False)
        ms = ctx.max_over_ranks([e0.elapsed_time(e1)])[0]
        blocks.append(ms)
        stamps.append((w0, w1))
        total_ms += ms
        if total_ms >= min_seconds * 1e3 or len(blocks) >= 200:
            break
    launches = lib.launch_count() - launches0
    fam = {}
    for name, f in (("decode", capi.KERNEL_DECODE), ("append", capi.KERNEL_APPEND), ("prefill", capi.KERNEL_PREFILL)):
        ms, n = lib.profile_read(f)
        fam[name] = (ms / max(n, 1), n)
    kms = ctx.max_over_ranks([fam["decode"][0], fam["append"][0], fam["prefill"][0]])
    return {"first_block_ms": blocks[0], "blocks": len(blocks), "all_ms": total_ms, "steps_per_block": steps,
            "first_block_wall": stamps[0], "whole_wall": (stamps[0][0], stamps[-1][1]),
            "launches_per_step": launches / (steps * len(blocks)),
            "kernel_ms": dict(zip(("decode", "append", "prefill"), kms)),
            "kernel_launches_timed": {k: v[1] for k, v in fam.items()}}


def kernel_rooflines(ctx: Ctx, dc, spec, idx, t, median_mhz=None):
    """Roofline entries of the decode and prefill kernels from the event-timed launches of a run."""
    from ppl_nn_b200 import workloads
    nd = idx.decoding_batches
    pk = ctx.peaks
    out = {}
    if t["kernel_launches_timed"]["decode"]:
        algo = workloads.decode_bytes(dc.num_kv_heads, spec.head_dim, idx.kvlens[:nd], dc.num_heads)
        ms = t["kernel_ms"]["decode"]
        ach = algo / (ms * 1e-3) / 1e9
        out["decode_splitk_kernel"] = {
            "bound": "hbm", "kernel": "decode_splitk_kernel", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": ach / pk["hbm_gbs"], "peak_source": pk["source"], "frac_of_nominal_8TBs": ach / 8000.0,
            "algorithmic_bytes_per_launch": algo, "kernel_ms": ms,
            "launches_timed": t["kernel_launches_timed"]["decode"], "per_gpu": True,
            "traffic": DECODE_TRAFFIC_PER_ALGO_BYTE * algo}
        if median_mhz:
            out["decode_splitk_kernel"]["kernel_ms_x_sm_mhz"] = ms * median_mhz
    if t["kernel_launches_timed"]["prefill"]:
        flops = workloads.prefill_flops(dc.num_heads, spec.head_dim, idx.seqlens[nd:])
        ms = t["kernel_ms"]["prefill"]
        ach = flops / (ms * 1e-3) / 1e12
        out["prefill_tcgen05_kernel"] = {
            "bound": "tensor", "kernel": "prefill_tcgen05_kernel", "achieved": ach, "peak": pk["tflops"],
            "unit": "TFLOP/s", "frac": ach / pk["tflops"], "peak_source": pk["source"],
            "frac_of_sustained_peak": ach / pk["tflops_sustained"], "algorithmic_flops_per_launch": flops,
            "kernel_ms": ms, "launches_timed": t["kernel_launches_timed"]["prefill"], "per_gpu": True, "traffic": None}
    return out


def shard_check(ctx: Ctx, spec, out, layout, page_size, heads=None):
    """Gather the shards' outputs (NCCL, untimed) and recompute a few kv heads on rank 0 as one-head workloads
    (the values of a head do not depend on the sharding): the gathered columns must agree within the
    operator's tolerance.  Returns a dict for the JSON line."""
    from ppl_nn_b200 import workloads
    torch, dist = ctx.torch, ctx.dist
    full = out
    if ctx.world > 1:
        parts = [torch.empty_like(out) for _ in range(ctx.world)]
        dist.all_gather(parts, out)
        full = torch.cat(parts, dim=1)
    res = {"output_abs_mean": float(full.float().abs().mean().item()), "gathered_heads": int(full.shape[1])}
    if ctx.rank != 0:
        return res
    assert full.shape[1] == spec.num_heads and bool(torch.isfinite(full.float()).all())
    group = spec.num_heads // spec.num_kv_heads
    heads = heads if heads is not None else sorted({0, spec.num_kv_heads - 1})
    worst = 0.0
    for h in heads:
        dc1 = workloads.device_case(spec, ctx.dev, rank=h, world=spec.num_kv_heads, layout=layout, page_size=page_size)
        i1 = dc1.index
        op1 = make_op(dc1, spec, layout, page_size)
        ref = op1.forward(dc1.query, dc1.current_key, dc1.current_value, dc1.seqstarts, dc1.kvstarts, dc1.cachestarts,
                          dc1.start_pos, i1.decoding_batches, i1.max_seqlen, i1.max_kvlen, dc1.cache, dc1.scale)
        if op1.device_status() != 0:
            raise SystemExit("device status word is not clean in the shard check")
        err = (ref.float() - full[:, h * group:(h + 1) * group].float()).abs().max().item()
        worst = max(worst, float(err))
        del dc1, op1, ref
        torch.cuda.empty_cache()
    if not worst <= 2e-3:
        raise SystemExit(f"shard check failed: recomputed kv heads {heads} differ by {worst:.3e} from the gathered output")
    res.update({"recomputed_kv_heads": heads, "max_abs_vs_one_head_recomputation": worst, "tolerance": 2e-3})
    return res


def run_config(ctx: Ctx, name: str, cache_prefill: bool, steps: int, warmup: int):
    """One of the other benchmark configurations, sharded over the ranks like the headline one."""
    from ppl_nn_b200 import workloads
    torch = ctx.torch
    spec = workloads.SPECS[name]
    if spec.num_kv_heads % ctx.world:
        return {"workload": name, "skipped": f"{spec.num_kv_heads} kv heads do not divide over {ctx.world} ranks"}
    dc = workloads.device_case(spec, ctx.dev, rank=ctx.rank, world=ctx.world)
    idx = dc.index
    nd = idx.decoding_batches
    op = make_op(dc, spec, 0, 0, cache_prefill)
    out = torch.empty_like(dc.query)
    fwd = (dc.query, dc.current_key, dc.current_value, dc.seqstarts, dc.kvstarts, dc.cachestarts, dc.start_pos, nd,
           idx.max_seqlen, idx.max_kvlen, dc.cache, dc.scale)
    t = timed_steps(ctx, lambda: op.forward(*fwd, attn_output=out), steps, warmup)
    status = op.device_status()
    ms = t["first_block_ms"] / steps
    roof = kernel_rooflines(ctx, dc, spec, idx, t)
    res = {"workload": name, "enable_cache_prefill": bool(cache_prefill), "n_gpus": ctx.world, "steps": steps,
           "decode_scores": decode_scores_form(spec),
           "sharding": f"kv-heads/{ctx.world}", "ms_per_step": ms, "tokens_per_step": int(idx.total_tokens),
           "decode_tokens_per_s": nd / (ms * 1e-3), "tokens_per_s": idx.total_tokens / (ms * 1e-3),
           "decode_sequences": nd, "kv_tokens": int(idx.kvlens[:nd].sum()), "prefill_sequences": idx.batch - nd,
           "prefill_tokens": int(idx.seqlens[nd:].sum()), "append_kernel_ms": t["kernel_ms"]["append"],
           "launches_per_step": t["launches_per_step"], "device_status": int(status), "kernels": roof,
           "output_abs_mean": float(out.float().abs().mean().item())}
    del dc, op, out, fwd
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--layout", type=int, default=0, choices=[0, 3])
    ap.add_argument("--page-size", type=int, default=0, help="paged cache (cache_mode 1) with pages of this many tokens")
    ap.add_argument("--seq-scale", type=float, default=1.0, help="fraction of the sequences (profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-per-config", action="store_true")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--cpu-seqs", type=int, default=32, help="sequences in the bounded CPU sample")
    ap.add_argument("--per-config-steps", type=int, default=30)
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        run_reference_arm(args, int(os.environ.get("RANK", "0")))
        return

    ctx = Ctx(args)
    torch, dist, lib, dev, rank, world = ctx.torch, ctx.dist, ctx.lib, ctx.dev, ctx.rank, ctx.world
    from ppl_nn_b200 import workloads

    spec = workloads.SPECS[args.workload]
    if args.seq_scale != 1.0:
        spec = workloads.scaled(spec, seqs=args.seq_scale)
    dc = workloads.device_case(spec, dev, rank=rank, world=world, layout=args.layout, page_size=args.page_size)
    idx = dc.index
    nd = idx.decoding_batches
    op = make_op(dc, spec, args.layout, args.page_size)
    out = torch.empty_like(dc.query)
    fwd_args = (dc.query, dc.current_key, dc.current_value, dc.seqstarts, dc.kvstarts, dc.cachestarts, dc.start_pos,
                nd, idx.max_seqlen, idx.max_kvlen, dc.cache, dc.scale)

    def step():
        op.forward(*fwd_args, attn_output=out)

    with ClockSampler(ctx.local_rank) as clocks:
        # ---- device-resident timing: W warm-ups, then exactly K steps; then the sustained repetition -------
        t = timed_steps(ctx, step, args.steps, args.warmup)
        status = op.device_status()
        if status != 0:
            raise SystemExit(f"device status word {status} after the timed steps")
        sus = None if args.no_sustained else timed_steps(ctx, step, args.steps, 0, min_seconds=0.5)
    ms_step = t["first_block_ms"] / args.steps
    tokens_per_step = idx.total_tokens  # new tokens of the step: one per decode sequence plus every prefill token
    value = tokens_per_step / (ms_step * 1e-3)
    clk = clocks.summary(*t["first_block_wall"])
    kernels = kernel_rooflines(ctx, dc, spec, idx, t, clk.get("sm_mhz"))
    dominant = max(kernels.values(), key=lambda k: k["kernel_ms"]) if kernels else None
    roofline = dict(dominant) if dominant else None
    if roofline is not None:
        roofline["append_kernel_ms"] = t["kernel_ms"]["append"]
        roofline["other_kernels"] = [k for k in kernels.values() if k is not dominant]
    sustained = None
    if sus is not None:
        sclk = clocks.summary(*sus["whole_wall"])
        sk = kernel_rooflines(ctx, dc, spec, idx, sus, sclk.get("sm_mhz"))
        sms = sus["all_ms"] / (sus["blocks"] * args.steps)
        sustained = {"steps": sus["blocks"] * args.steps, "seconds": sus["all_ms"] * 1e-3, "ms_per_step": sms,
                     "value": tokens_per_step / (sms * 1e-3), "unit": "tokens/s", "clocks": sclk,
                     "roofline": sk.get(dominant["kernel"]) if dominant else None}

    # ---- end to end: host buffers in, host buffer out, every step -------------------------------
    e2e = None
    if not args.no_e2e:
        # The step's seven input tensors live back to back in ONE pinned host buffer and ONE device buffer
        # (256-byte aligned views), so a step's inputs cross the bus as a single copy.
        names = ("query", "current_key", "current_value", "seqstarts", "kvstarts", "cachestarts", "start_pos")
        offs, total = {}, 0
        for k in names:
            x = getattr(dc, k)
            offs[k] = total
            total += (x.numel() * x.element_size() + 255) // 256 * 256
        stage_host = torch.empty(total, dtype=torch.uint8).pin_memory()
        stage_dev = torch.empty(total, dtype=torch.uint8, device=dev)

        def view(buf, k):
            x = getattr(dc, k)
            n = x.numel() * x.element_size()
            return buf[offs[k]:offs[k] + n].view(x.dtype).view(x.shape)

        host = {k: view(stage_host, k) for k in names}
        devbuf = {k: view(stage_dev, k) for k in names}
        for k in names:
            host[k].copy_(getattr(dc, k).cpu())
        out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        h2d = sum(v.numel() * v.element_size() for v in host.values())
        d2h = out_host.numel() * out_host.element_size()

        # the reference-facing route: the C++ Op/Kernel pair created through the registry, fed the
        # operator's 12 inputs (scalars as host tensors); its workspace comes from the engine's pool
        from ppl_nn_b200 import hostapi
        hostapi.register_ops()
        eng = hostapi.Engine(ctx.local_rank, torch.cuda.current_stream().cuda_stream)
        paging = dict(cache_mode=1, page_size=args.page_size) if args.page_size else {}
        hop = hostapi.Op(eng, "MultiHeadCacheAttention",
                         dict(num_heads=dc.num_heads, num_kv_heads=dc.num_kv_heads, head_dim=spec.head_dim, num_layer=1,
                              layer_idx=0, quant_bit=8, quant_group=8, cache_layout=args.layout, **paging))
        hin = [hostapi.describe(x)[0] for x in
               (devbuf["query"], devbuf["current_key"], devbuf["current_value"], devbuf["seqstarts"],
                devbuf["kvstarts"], devbuf["cachestarts"], devbuf["start_pos"])]
        scal = [np.array(v, dtype=np.int64) for v in (nd, idx.max_seqlen, idx.max_kvlen)]
        hin += [hostapi.describe(v)[0] for v in scal]
        hin += [hostapi.describe(dc.cache)[0], hostapi.describe(dc.scale)[0]]
        hout = [hostapi.describe(out)[0]]

        run_op, _ = hop.bind(hin, hout)  # the argument arrays are built once, like a serving loop would

        def e2e_step():
            stage_dev.copy_(stage_host, non_blocking=True)
            rc = run_op()
            if rc != "RC_SUCCESS":
                raise SystemExit(f"MultiHeadCacheAttention kernel returned {rc}")
            out_host.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the caller reads the result before the next step

        for _ in range(args.warmup):
            e2e_step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        ctx.barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = ctx.max_over_ranks([max(e0.elapsed_time(e1), 0.0)])[0]
        e2e = {"value": tokens_per_step / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms / args.steps,
               "wall_ms_per_step": wall_ms / args.steps,
               "api": "host-layer DynamicBatchingMultiHeadCacheAttentionKernel::Execute via the op registry (C ABI below)"}
        step()  # leave `out` as the device-resident path computes it

    # ---- correctness of the sharded run: gather (NCCL, outside every timed region) + recomputation ----
    torch.cuda.synchronize(dev)
    check = shard_check(ctx, spec, out, args.layout, args.page_size) if nd == idx.batch else \
        {"output_abs_mean": float(out.float().abs().mean().item())}

    # ---- the other configurations, same ranks ------------------------------------------------------
    config_bits = dict(num_heads=spec.num_heads, num_kv_heads=spec.num_kv_heads, head_dim=spec.head_dim,
                       decode_sequences=nd, kv_tokens=int(idx.kvlens[:nd].sum()), prefill_sequences=idx.batch - nd,
                       prefill_tokens=int(idx.seqlens[nd:].sum()))
    algo_bytes = workloads.decode_bytes(dc.num_kv_heads, spec.head_dim, idx.kvlens[:nd], dc.num_heads) if nd else 0
    del dc, op, fwd_args
    if not args.no_e2e:
        del devbuf, stage_dev, hin, hout, run_op, hop
    torch.cuda.empty_cache()
    per_config = None
    if not args.no_per_config:
        per_config = [run_config(ctx, name, cp, args.per_config_steps, 5) for name, cp in PER_CONFIG]

    # ---- CPU baseline on a bounded sample (rank 0, single-GPU run only) -------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and nd == idx.batch:
        cpu = cpu_time_sample(workloads.SPECS[args.workload], args.cpu_seqs)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": spec.name, **config_bits,
                       "cache_layout": args.layout, "page_size": args.page_size, "sharding": f"kv-heads/{world}",
                       "decode_scores": decode_scores_form(spec),
                       "l2": "no flush: the per-GPU cache working set is far larger than the 126 MB L2"
                             if algo_bytes > 4 * 126e6 else
                             "no flush: the step is compute-bound prefill" if nd == 0 else
                             "working set is NOT much larger than L2"},
            "hbm_gbs_per_gpu_whole_step": algo_bytes / (ms_step * 1e-3) / 1e9,
            "tokens_per_step": int(tokens_per_step),
            "roofline": roofline, "sustained": sustained, "cpu_baseline": cpu, "clocks": clk, "e2e": e2e,
            "gpu_launches": int(round(t["launches_per_step"] * args.steps)),
            "gpu_launches_per_step": t["launches_per_step"],
            "output_abs_mean": check["output_abs_mean"], "shard_check": check, "device_status": int(status),
            "per_config": per_config,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _run_with_clean_stdout():
    """Everything but the final JSON line goes to stderr: libraries (NCCL prints its version banner to
    stdout, for one) must not add lines to the one-line contract."""
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    lines = []
    real_print = print

    def capture(*a, **kw):
        if kw.get("file") in (None, sys.stdout):
            lines.append(" ".join(str(x) for x in a))
        else:
            real_print(*a, **kw)

    import builtins
    builtins.print = capture
    try:
        main()
    finally:
        builtins.print = real_print
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)
    for ln in lines:
        real_print(ln, flush=True)


if __name__ == "__main__":
    _run_with_clean_stdout()
