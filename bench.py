#!/usr/bin/env python
"""Benchmark of the INT8-KV cache attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One *step* is one call of the MultiHeadCacheAttention operator (quantise-and-append of the new
token of every sequence, then ragged split-k decode attention over the INT8 cache) on one
transformer layer.  The default workload is the LLaMA-2-7B pure-decode configuration: 256
sequences, MHA 32 heads x 128, KV lengths uniform in [128, 4096], seed 1, N(0,1) values with
every 16th K channel scaled by 8; the cache is 5.6 GB, far larger than the 126 MB L2, so no
flush is needed between steps.  With N > 1 the KV heads (and their query heads) are sharded over
the ranks exactly like tensor parallelism shards them; there is no collective in the timed path
(an all-gather of the outputs afterwards is only a sanity check), total work is fixed, so the
run is a strong-scaling run.

Rank 0 prints ONE JSON line.  `value` is decode tokens per second of the whole job with all
inputs resident in HBM; `e2e` is the same metric through the reference-facing operator (the C++ Op/Kernel
classes of ppl.nn_b200/host, created via the registry) with HOST
inputs (pinned host -> device copies of query/key/value and the index tensors, device -> host
copy of the attention output, every step, inside the timed region; the KV cache itself is
device-resident state by the operator's contract).  `roofline` is for the dominant kernel
(decode_splitk_kernel), timed with CUDA events on its own stream inside the library.
`cpu_baseline` is the CPU restatement of the reference's path (oracle/kvattn_oracle.c, OpenMP)
on the host cores of the same machine.

`--impl reference` times that CPU restatement alone (the reference's CUDA kernels are not part
of its source tree and nothing of it builds here), on a bounded sample of the same workload.
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

# DRAM bytes moved by decode_splitk_kernel per algorithmic byte, from the ncu capture summarised in
# profiles/ (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the captured
# launch): 692.67 MB + 5.64 MB for 690.86 MB (profiles/decode_splitk_kernel_cfg2_eighth.md).
DECODE_TRAFFIC_PER_ALGO_BYTE = 1.0108


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs, copy read+write)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


def measured_peak_tflops():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, cuBLAS burst)"
        except Exception:
            pass
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def measured_sustained_tflops():
    """cuBLAS bf16 over a seconds-long loop under the power cap: the yardstick for a kernel inside a long step."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops_sustained"])
        except Exception:
            pass
    return 1400.0


# ------------------------------------------------------------------------------------------------
# clocks: NVML samples taken while the timed region runs (read-only)
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, device_index: int, period_s: float = 0.005):
        self.samples, self.reasons, self.power_w, self.mem_mhz = [], set(), [], []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            # map the CUDA device to NVML through its PCI bus id
            import torch
            bus = torch.cuda.get_device_properties(device_index).pci_bus_id \
                if hasattr(torch.cuda.get_device_properties(device_index), "pci_bus_id") else None
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
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                self.mem_mhz.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_MEM)))
                self.power_w.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
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

    def summary(self):
        if self._h is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": getattr(self, "error", "no NVML")}
        return {"sm_mhz": int(statistics.median(self.samples)) if self.samples else None,
                "sm_min_mhz": min(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples),
                "mem_mhz": int(statistics.median(self.mem_mhz)) if self.mem_mhz else None,
                "power_w_max": round(max(self.power_w), 1) if self.power_w else None}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle port on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_time_sample(spec, num_seqs: int, target_seconds: float = 12.0, steps: int | None = None, warmup: int = 1):
    """Time the CPU restatement on the first `num_seqs` decode sequences of `spec` (same seeded
    lengths).  Cache contents are random valid codes/scales: the arithmetic does not depend on
    them.  With `steps` the run is exactly `warmup` + `steps` passes and the sample shrinks (fewer
    sequences) until that fits about a minute and a half; without it the number of passes is chosen to
    fill `target_seconds`.  Returns (tokens_per_s, cores, seconds_per_step, steps, sample_text)."""
    from ppl_nn_b200 import workloads
    om = entry.load_oracle()
    orc = om.COracle()
    kv_all, _ = workloads.draw_lengths(spec)
    rng = np.random.default_rng(99)
    Hq, Hkv, Dh = spec.num_heads, spec.num_kv_heads, spec.head_dim

    def make(n):
        kv = kv_all[:n]
        idx = workloads.make_index(kv, [])
        cshape, sshape = workloads.cache_shapes(0, idx.max_tokens, 1, Hkv, Dh)
        cache = rng.integers(-127, 128, size=cshape, dtype=np.int8)
        scale = rng.uniform(0.01, 0.05, size=sshape).astype(np.float16)
        T = idx.total_tokens
        q = rng.standard_normal((T, Hq, Dh), dtype=np.float32).astype(np.float16)
        ck = rng.standard_normal((T, Hkv, Dh), dtype=np.float32).astype(np.float16)
        cv = rng.standard_normal((T, Hkv, Dh), dtype=np.float32).astype(np.float16)
        d = orc.desc(num_heads=Hq, num_kv_heads=Hkv, head_dim=Dh, batch=idx.batch, decoding_batches=idx.batch,
                     max_tokens=idx.max_tokens)
        return kv, idx, (lambda: orc.mhca(d, q, ck, cv, idx.seqstarts, idx.cachestarts, idx.start_pos, cache, scale))

    kv, idx, step = make(num_seqs)
    t0 = time.perf_counter()
    step()  # first pass: warms up, and tells us how long a step is
    one = time.perf_counter() - t0
    if steps is None:
        steps = max(1, min(50, int(target_seconds / max(one, 1e-4))))
    else:
        budget = 90.0
        done = 1
        if one * (steps + warmup) > budget and num_seqs > 4:
            num_seqs = max(4, int(num_seqs * budget / (one * (steps + warmup))))
            kv, idx, step = make(num_seqs)
            done = 0
        for _ in range(max(warmup - done, 0)):
            step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    per_step = (time.perf_counter() - t0) / steps
    cores = orc.num_threads()
    sample = (f"first {idx.batch} of {spec.n_decode} sequences of {spec.name} (same seeded KV lengths, "
              f"{int(kv.sum())} cached tokens), append + decode attention, {steps} steps, OpenMP x{cores}")
    return idx.batch / per_step, cores, per_step, steps, sample


def run_reference_arm(args, rank: int):
    """`--impl reference`: the reference's CUDA kernels are absent from its tree and nothing of it
    compiles here, so this arm is the CPU restatement of its path on all host threads."""
    if rank != 0:
        return
    entry.load_package()
    from ppl_nn_b200 import workloads
    spec = workloads.SPECS[args.workload]
    nseq = min(spec.n_decode, args.cpu_seqs)
    # one "step" of this arm = one pass over the bounded sample; K steps after W warm-ups
    om = entry.load_oracle()
    om.build()
    tok_s, cores, per_step, steps, sample = cpu_time_sample(spec, nseq, steps=args.steps, warmup=max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": max(args.warmup, 1), "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp16 in/out, int8 cache, fp32 accumulate", "data": "synthetic",
        "config": {"workload": spec.name, "sample": sample},
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference path (oracle/kvattn_oracle.c); the reference's own kernels live "
                "in the un-vendored ppl.llm.kernel.cuda and do not exist in its tree",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
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
    ap.add_argument("--cpu-seqs", type=int, default=64, help="sequences in the bounded CPU sample")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")

    import torch
    import torch.distributed as dist
    entry.load_package()
    from ppl_nn_b200 import capi, ops, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    lib = capi.library()
    if not lib.device_ready():
        raise SystemExit("the CUDA library has no sm_100a code for this device")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    spec = workloads.SPECS[args.workload]
    if args.seq_scale != 1.0:
        spec = workloads.scaled(spec, seqs=args.seq_scale)
    dc = workloads.device_case(spec, dev, rank=rank, world=world, layout=args.layout, page_size=args.page_size)
    idx = dc.index
    nd = idx.decoding_batches
    paging = dict(cache_mode=1, page_size=args.page_size) if args.page_size else {}
    op = ops.MultiHeadCacheAttention(
        ops.MultiHeadCacheAttentionParam(num_heads=dc.num_heads, num_kv_heads=dc.num_kv_heads, head_dim=spec.head_dim,
                                         num_layer=1, layer_idx=0, quant_bit=8, cache_layout=args.layout, **paging))
    out = torch.empty_like(dc.query)
    fwd_args = (dc.query, dc.current_key, dc.current_value, dc.seqstarts, dc.kvstarts, dc.cachestarts, dc.start_pos,
                nd, idx.max_seqlen, idx.max_kvlen, dc.cache, dc.scale)

    def step():
        op.forward(*fwd_args, attn_output=out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident timing: W warm-ups, then exactly K steps -----------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    status = op.device_status()
    if status != 0:
        raise SystemExit(f"device status word {status} after warm-up")
    launches0 = lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # the library brackets the kernels of timed steps with its own event pairs (on the launching stream),
    # so the dominant kernel's duration comes from launches of the timed region itself
    lib.profile_read(capi.KERNEL_DECODE)
    lib.profile_read(capi.KERNEL_APPEND)
    lib.profile_read(capi.KERNEL_PREFILL)
    # Every fourth timed step is bracketed (four event records cost a few microseconds, which shows on a
    # 150 us step of an 8-way shard); the others run exactly as a caller would run them.
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for i in range(args.steps):
            lib.profile_enable(i % 4 == 0)
            step()
        e1.record()
        barrier()
    lib.profile_enable(False)
    launches = lib.launch_count() - launches0
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    tokens_per_step = idx.total_tokens  # new tokens of the step: one per decode sequence plus every prefill token
    value = tokens_per_step / (ms_step * 1e-3)

    dec_ms, dec_n = lib.profile_read(capi.KERNEL_DECODE)
    app_ms, app_n = lib.profile_read(capi.KERNEL_APPEND)
    pre_ms, pre_n = lib.profile_read(capi.KERNEL_PREFILL)
    times = {"decode": dec_ms / max(dec_n, 1), "append": app_ms / max(app_n, 1), "prefill": pre_ms / max(pre_n, 1)}
    if world > 1:
        t = torch.tensor([times["decode"], times["append"], times["prefill"]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = dict(zip(("decode", "append", "prefill"), (float(v) for v in t.tolist())))
    algo_bytes = workloads.decode_bytes(dc.num_kv_heads, spec.head_dim, idx.kvlens[:nd], dc.num_heads) if nd else 0
    algo_flops = workloads.prefill_flops(dc.num_heads, spec.head_dim, idx.seqlens[nd:])
    peak, peak_src = measured_peak_gbs()
    tpeak, tpeak_src = measured_peak_tflops()
    kernels = {}
    if dec_n:
        ach = algo_bytes / (times["decode"] * 1e-3) / 1e9
        kernels["decode_splitk_kernel"] = {
            "bound": "hbm", "kernel": "decode_splitk_kernel", "achieved": ach, "peak": peak, "unit": "GB/s",
            "frac": ach / peak, "peak_source": peak_src, "frac_of_nominal_8TBs": ach / 8000.0,
            "algorithmic_bytes_per_launch": algo_bytes, "kernel_ms": times["decode"], "launches_timed": dec_n,
            "per_gpu": True,
            "traffic": (DECODE_TRAFFIC_PER_ALGO_BYTE * algo_bytes) if DECODE_TRAFFIC_PER_ALGO_BYTE else None}
    if pre_n:
        ach = algo_flops / (times["prefill"] * 1e-3) / 1e12
        kernels["prefill_tcgen05_kernel"] = {
            "bound": "tensor", "kernel": "prefill_tcgen05_kernel", "achieved": ach, "peak": tpeak, "unit": "TFLOP/s",
            "frac": ach / tpeak, "peak_source": tpeak_src, "frac_of_sustained_peak": ach / measured_sustained_tflops(),
            "algorithmic_flops_per_launch": algo_flops,
            "kernel_ms": times["prefill"], "launches_timed": pre_n, "per_gpu": True, "traffic": None}
    dominant = max(kernels.values(), key=lambda k: k["kernel_ms"]) if kernels else None
    roofline = dict(dominant) if dominant else None
    if roofline is not None:
        roofline["append_kernel_ms"] = times["append"]
        roofline["other_kernels"] = [k for k in kernels.values() if k is not dominant]

    # ---- end to end: host buffers in, host buffer out, every step -------------------------------
    e2e = None
    if not args.no_e2e:
        # The step's seven input tensors live back to back in ONE pinned host buffer and ONE device buffer
        # (256-byte aligned views), so a step's inputs cross the bus as a single copy.
        names = ("query", "current_key", "current_value", "seqstarts", "kvstarts", "cachestarts", "start_pos")
        offs, total = {}, 0
        for k in names:
            t = getattr(dc, k)
            offs[k] = total
            total += (t.numel() * t.element_size() + 255) // 256 * 256
        stage_host = torch.empty(total, dtype=torch.uint8).pin_memory()
        stage_dev = torch.empty(total, dtype=torch.uint8, device=dev)

        def view(buf, k):
            t = getattr(dc, k)
            n = t.numel() * t.element_size()
            return buf[offs[k]:offs[k] + n].view(t.dtype).view(t.shape)

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
        eng = hostapi.Engine(local_rank, torch.cuda.current_stream().cuda_stream)
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
        barrier()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = max(e0.elapsed_time(e1), 0.0)
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": tokens_per_step / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms / args.steps,
               "wall_ms_per_step": wall_ms / args.steps, "api": "host-layer DynamicBatchingMultiHeadCacheAttentionKernel::Execute via the op registry (C ABI below)"}

    # ---- sanity: gather the head shards (NCCL, outside every timed region) ----------------------
    checksum = float(out.float().abs().mean().item())
    if world > 1:
        parts = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(parts, out)
        full = torch.cat(parts, dim=1)
        assert full.shape[1] == spec.num_heads and bool(torch.isfinite(full.float()).all())
        checksum = float(full.float().abs().mean().item())

    # ---- CPU baseline on a bounded sample (rank 0, single-GPU run only) -------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and nd == idx.batch:
        entry.load_oracle().build()
        base_spec = workloads.SPECS[args.workload]
        tok_s, cores, per_step, steps, sample = cpu_time_sample(base_spec, min(base_spec.n_decode, args.cpu_seqs))
        cpu = {"value": tok_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
               "ms_per_step_of_sample": per_step * 1e3}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp16 in/out, int8 cache, fp32 accumulate", "data": "synthetic",
            "config": {"workload": spec.name, "num_heads": spec.num_heads, "num_kv_heads": spec.num_kv_heads,
                       "head_dim": spec.head_dim, "decode_sequences": nd, "kv_tokens": int(idx.kvlens[:nd].sum()),
                       "prefill_sequences": idx.batch - nd, "prefill_tokens": int(idx.seqlens[nd:].sum()),
                       "cache_layout": args.layout, "page_size": args.page_size, "sharding": f"kv-heads/{world}",
                       "l2": "no flush: the per-GPU cache working set is far larger than the 126 MB L2"
                             if algo_bytes > 4 * 126e6 else
                             "no flush: the step is compute-bound prefill" if nd == 0 else
                             "working set is NOT much larger than L2"},
            "hbm_gbs_per_gpu_whole_step": algo_bytes / (ms_step * 1e-3) / 1e9,
            "tokens_per_step": int(tokens_per_step),
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks.summary(), "e2e": e2e,
            "gpu_launches": int(launches), "output_abs_mean": checksum, "device_status": int(status),
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
