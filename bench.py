#!/usr/bin/env python
"""Benchmark of the Flash-MSA training hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c5]

One step = one forward + backward of ``flash_msa_func`` (block scoring, top-k, reverse index, sparse
forward with combine, fused backward, casts) on synthetic N(0,1) bf16 inputs of the benchmark
configuration "c2": B=2, S=8192, Hq=32, Hkv=8, Hp=8, Hpkv=8, D=128, top_k=16 blocks, causal.
With N GPUs every rank runs its own c2-sized shard of a global batch of 2N (the path shards by
(batch, KV-head group) with no collective), so scaling is weak and ``value`` is the aggregate.

Metric: TFLOP/s on the effective (selected-block) FLOPs  F = 7 * 2*D * pairs(S,Kb) * B * Hq
(2 forward + 5 backward products over the unmasked selected pairs; recompute, proxy work and
padding are not counted).  Timing: CUDA events on the launching stream, barrier +
synchronize on both sides, max over ranks.  Inputs (>400 MB per step) exceed the 126 MB L2, so no
explicit flush is needed.

``--impl reference`` times the reference algorithm on the host cores instead: the oracle's
restatement of the reference's eager model (fp32, all torch threads) on one (batch, KV-head group)
slice of the same workload per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, S, Hq, Hkv, Hp, Hpkv, Kb, warmup-mode)
    "c2": dict(b=2, s=8192, hq=32, hkv=8, hp=8, hpkv=8, kb=16, dense=False,
               desc="sparse MSA fwd+bwd, B=2 S=8192 Hq=32 Hkv=8 Hp=8 Hpkv=8 D=128 top_k=16 blocks, causal, N(0,1) bf16"),
    # a quarter of c2 (same S, top_k and head ratios): the small case used for ncu captures
    "c2q": dict(b=1, s=8192, hq=16, hkv=4, hp=4, hpkv=4, kb=16, dense=False,
                desc="sparse MSA fwd+bwd, quarter of c2: B=1 S=8192 Hq=16 Hkv=4 Hp=4 Hpkv=4 D=128 top_k=16 blocks"),
    "c3": dict(b=4, s=4096, hq=32, hkv=8, hp=8, hpkv=8, kb=1, dense=True,
               desc="MSA warmup fwd+bwd, B=4 S=4096 Hq=32 Hkv=8 Hp=8 Hpkv=8 D=128, dense causal + proxy KL"),
    "c5": dict(b=1, s=65536, hq=64, hkv=8, hp=16, hpkv=8, kb=32, dense=False,
               desc="long-context sparse MSA, B=1 S=65536 Hq=64 Hkv=8 Hp=16 Hpkv=8 top_k=32 blocks, sharded by KV group"),
}
SCALE = 128 ** -0.5
# DRAM bytes per launch of the dominant kernel (sparse backward at c2): dram__bytes_read.sum +
# dram__bytes_write.sum of the ncu capture summarised in profiles/sparse_bwd_kernel_c2q.md (a quarter-size
# case), scaled by 4 to the full launch.
BWD_TRAFFIC_BYTES_C2 = 4 * (285.179904e6 + 618.938624e6)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": p["bf16_tflops"], "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


def flops(cfg):
    from oracle.msa_oracle import flops_sparse_fwd_bwd, flops_warmup_fwd_bwd
    if cfg["dense"]:
        return flops_warmup_fwd_bwd(cfg["b"], cfg["s"], cfg["hq"])
    return flops_sparse_fwd_bwd(cfg["b"], cfg["s"], cfg["hq"], cfg["kb"])


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs (read-only
    NVML queries from a background thread, every few milliseconds; nvidia-smi polling as the fallback)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.file = None
        self.thread = None
        self.stop_flag = False
        self.sm, self.mx, self.reasons = [], [], set()

    def _nvml_loop(self, nv, handle):
        masks = [("hw_slowdown", nv.nvmlClocksThrottleReasonHwSlowdown),
                 ("hw_thermal_slowdown", nv.nvmlClocksThrottleReasonHwThermalSlowdown),
                 ("sw_thermal_slowdown", nv.nvmlClocksThrottleReasonSwThermalSlowdown),
                 ("sw_power_cap", nv.nvmlClocksThrottleReasonSwPowerCap)]
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                for name, m in masks:
                    if bits & m:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        try:
            import threading

            import pynvml as nv
            nv.nvmlInit()
            # NVML numbers devices like nvidia-smi; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [x for x in vis.split(",") if x.strip().isdigit()]
            phys = int(ids[self.index]) if self.index < len(ids) else self.index
            handle = nv.nvmlDeviceGetHandleByIndex(phys)
            self.mx.append(float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": max(self.mx) if self.mx else None,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


# --------------------------------------------------------------------------------------------
# CPU arm (reference algorithm on the host cores)
# --------------------------------------------------------------------------------------------
def cpu_slice_step(cfg, tensors):
    """One fwd+bwd of the reference's eager algorithm on one (batch, KV group) slice."""
    from oracle import msa_oracle as O
    qp, kp, q, k, v, do = tensors
    if cfg["dense"]:
        fn = lambda *t: O.eager_warmup(*t, SCALE)
    else:
        fn = lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE)
    O.eager_forward_backward(fn, (qp, kp, q, k, v), do, 1.0)


def cpu_slice(cfg, seed=0):
    """Slice geometry: one batch element, one KV head with its main and proxy heads."""
    from oracle import msa_oracle as O
    g = cfg["hq"] // cfg["hkv"]
    ppk = cfg["hp"] // cfg["hkv"]
    pkv = max(1, cfg["hpkv"] // cfg["hkv"])
    tensors = O.make_inputs(1, cfg["s"], g, 1, ppk, min(pkv, ppk), seed=seed)
    slices = cfg["b"] * cfg["hkv"]
    sl = dict(cfg, b=1, hq=g)
    return tensors, slices, flops(sl)


def run_cpu_baseline(cfg, steps, warmup):
    torch.set_num_threads(os.cpu_count() or 1)
    tensors, slices, f_slice = cpu_slice(cfg)
    for _ in range(warmup):
        cpu_slice_step(cfg, tensors)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_slice_step(cfg, tensors)
        times.append(time.perf_counter() - t0)
    t = sum(times) / len(times)
    return {"value": f_slice / t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 of {slices} (batch, KV-head group) slices of the workload per step "
                      f"(S={cfg['s']}, {cfg['hq'] // cfg['hkv']} main heads), fp32 eager restatement, {steps} step(s)",
            "s_per_slice": t, "slices": slices}


def reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = run_cpu_baseline(cfg, args.steps, args.warmup)
    per_slice = base.pop("s_per_slice")
    slices = base.pop("slices")
    line = {
        "impl": "reference", "metric": "sparse_attn_fwd_bwd_tflops", "value": base["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_slice * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["desc"], "l2": "inputs larger than L2"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": cfg["s"] / (per_slice * slices / cfg["b"]) if slices else None,
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------
# bandwidth kernels at long-context size (they are launch-latency dominated at c2)
# --------------------------------------------------------------------------------------------
def micro_select(args):
    """Achieved GB/s of the top-k pick and of the reverse index on materialised scores of the
    config-5 size (B*Hp = 16, S = 65536, NB = 512, top_k = 32 blocks).  Algorithmic bytes:
    top-k reads the causal half of the fp32 scores and writes Kb int32 per row; the reverse index
    reads block_indices twice and writes col_q, edge_pos and row_ptr."""
    from flash_msa_b200 import ops
    dev = torch.device("cuda", 0)
    rows_bh, s, kb = 16, 65536, 32
    nb = s // 128
    peaks = measured_peaks()
    gen = torch.Generator(device=dev).manual_seed(0)
    scores = torch.randn(1, rows_bh, s, nb, device=dev, generator=gen)
    idx = ops.select_topk(scores, kb)
    rix = ops.build_reverse_index(idx)
    torch.cuda.synchronize()
    edges = int(rix.row_ptr[-1].item())
    bytes_topk = rows_bh * sum((q // 128 + 1) for q in range(0, s, 128)) * 128 * 4 + rows_bh * s * kb * 4
    bytes_rix = 2 * rows_bh * s * kb * 4 + edges * 4 + rows_bh * s * kb * 4 + (rows_bh * nb + 1) * 4
    out = {}
    for name, fn, nbytes in (("select_topk", lambda: ops.select_topk(scores, kb), bytes_topk),
                             ("reverse_index", lambda: ops.build_reverse_index(idx), bytes_rix)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b in ev:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        ms = statistics.median(a.elapsed_time(b) for a, b in ev)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "algorithmic_bytes": nbytes, "GB/s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                     "peak_GB/s": peaks["hbm_gbs"], "peak_source": peaks["source"]}
    print(json.dumps({"micro": "select kernels at B*Hp=16 S=65536 top_k=32 blocks", "edges": edges, **out}))


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--micro-select", action="store_true", help="time the top-k and reverse-index kernels at config-5 size")
    args = ap.parse_args()
    if args.micro_select:
        micro_select(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)
    cfg = dict(WORKLOADS[args.workload])

    if args.impl == "reference":
        reference_arm(args, cfg)
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (flash_msa_b200 has no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    import flash_msa_b200
    from flash_msa_b200 import ops
    from flash_msa_b200.sharding import shard_workload
    from oracle.msa_oracle import make_inputs

    # strong-scaling workload (c5): one global problem split by KV group; others: one full problem per rank
    local = shard_workload(cfg, rank, world) if args.workload == "c5" else dict(cfg)
    scaling = "strong" if args.workload == "c5" else "weak"
    fn = flash_msa_b200.flash_msa_warmup_func if cfg["dense"] else flash_msa_b200.flash_msa_func
    top_k = cfg["kb"] * 128

    host = make_inputs(local["b"], local["s"], local["hq"], local["hkv"], local["hp"], local["hpkv"], seed=rank,
                       dtype=torch.bfloat16)
    host = [t.pin_memory() for t in host]
    devt = [t.to(dev) for t in host]
    qp, kp, q, k, v, do = devt
    ones = torch.ones((), device=dev)

    def step():
        leaves = [t.detach().requires_grad_(True) for t in (qp, kp, q, k, v)]
        out, kl = fn(*leaves, top_k, SCALE)
        torch.autograd.backward([out, kl], [do, ones])
        return out, [t.grad for t in leaves]

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()

    # ---- timed region: device-resident inputs ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ops.KERNEL_EVENTS = []
    launches0 = ops.LAUNCHES
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    start.record()
    for _ in range(args.steps):
        step()
    end.record()
    sync_all()
    elapsed_ms = start.elapsed_time(end)
    launches = ops.LAUNCHES - launches0
    events = ops.KERNEL_EVENTS
    ops.KERNEL_EVENTS = None
    clocks = sampler.stop() if rank == 0 else None
    per_kernel = {}
    for name, s, e in events:
        per_kernel.setdefault(name, []).append(s.elapsed_time(e))
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())

    # ---- end to end: host buffers, copies inside the timed region ----
    e2e = None
    if not args.no_e2e:
        # the repo's host-buffer call: pinned host tensors in, pinned host tensors out, copies and kernels
        # pipelined over (batch, KV-group) chunks on three streams (flash_msa_b200/host.py)
        from flash_msa_b200.host import HostStep
        hs = HostStep(local["b"], local["s"], local["hq"], local["hkv"], local["hp"], local["hpkv"], top_k, SCALE,
                      dense=cfg["dense"], device=dev)

        def e2e_step():
            return hs.run(*host, grad_kl=1.0)

        e2e_step()
        hs.synchronize()
        sync_all()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(2, min(args.steps, 5))
        s2.record()
        for _ in range(n_e2e):
            e2e_step()
        # the step ends when the last result has reached host memory
        torch.cuda.current_stream().wait_stream(hs.s_out)
        torch.cuda.current_stream().wait_stream(hs.s_cmp)
        e2.record()
        sync_all()
        e2e_ms = s2.elapsed_time(e2)
        if dist is not None:
            t = torch.tensor([e2e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        h2d, d2h = hs.bytes_per_step()
        total_f = flops(cfg) * (world if scaling == "weak" else 1)
        e2e = {"value": total_f * n_e2e / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / n_e2e, "steps": n_e2e}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    total_flops = flops(cfg) * (world if scaling == "weak" else 1)
    ms_per_step = elapsed_ms / args.steps
    value = total_flops / (ms_per_step * 1e-3) / 1e12
    tokens = cfg["b"] * cfg["s"] * (world if scaling == "weak" else 1)

    # dominant kernel: the fused backward.  Algorithmic FLOPs per launch = 5 products over the
    # selected pairs of this rank's problem.
    bwd_times = per_kernel.get("attn_bwd", [float("nan")])
    bwd_ms_step = sum(bwd_times) / args.steps            # all launches of one step (large problems run in passes)
    bwd_launches = len(bwd_times) / args.steps
    bwd_flops = flops(local) * 5.0 / 7.0
    achieved = bwd_flops / (bwd_ms_step * 1e-3) / 1e12
    traffic = BWD_TRAFFIC_BYTES_C2 if (args.workload == "c2" and bwd_launches == 1) else None
    roofline = {"kernel": "sparse_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "traffic": traffic,
                "peak_source": f"{peaks['source']} (burst cuBLAS bf16)", "ms_per_launch": bwd_ms_step / bwd_launches,
                "launches_per_step": bwd_launches}
    step_total = sum(sum(v) for v in per_kernel.values()) / args.steps
    breakdown = {n: {"ms_per_step": sum(v) / args.steps, "share": (sum(v) / args.steps) / step_total if step_total else None}
                 for n, v in sorted(per_kernel.items())}

    line = {
        "metric": "sparse_attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg["desc"], "sharding": "(batch, KV-head group), no collective on the kernel path",
                   "l2": "inputs larger than L2 (no flush needed)", "per_rank": local},
        "tokens_per_s": tokens / (ms_per_step * 1e-3),
        "frac_of_peak": value / (peaks["bf16_tflops"] * world),
        "roofline": roofline, "kernels": breakdown, "clocks": clocks, "gpu_launches": launches,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = {k_: v_ for k_, v_ in run_cpu_baseline(cfg, 1, 1).items() if k_ not in ("s_per_slice", "slices")}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
