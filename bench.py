#!/usr/bin/env python
"""Benchmark of the Flash-MSA training hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c2q|c3|c4b1|c5]

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

``e2e`` is the same step through ``flash_msa_b200.host.HostStep`` on pinned host buffers (copies in both directions
inside the timed region), with ``copy_floor_ms`` (the same copies alone) and ``device_allocs_in_timed_steps`` (cudaMalloc
calls of the caching allocator inside the timed steps; 0 in a steady pipeline) beside it.

``--impl reference`` times the reference algorithm on the host cores instead: the reference's own eager
model from the local copy under ``oracle/_ref`` (the oracle's restatement of it when that copy is absent), fp32, all
torch threads, on one (batch, KV-head group) slice of the same workload per step.
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
    # one batch element of config 4 (its B = 8 elements are independent): full length, full head set, skewed selection
    "c4b1": dict(b=1, s=32768, hq=48, hkv=4, hp=8, hpkv=4, kb=64, dense=False, skew=True,
                 desc="skewed-selection sparse MSA, one of the 8 batch elements of config 4: B=1 S=32768 Hq=48 Hkv=4 Hp=8 Hpkv=4 "
                      "top_k=64 blocks, block-mean keys + noise, Qp x4, sink blocks"),
    "c5": dict(b=1, s=65536, hq=64, hkv=8, hp=16, hpkv=8, kb=32, dense=False,
               desc="long-context sparse MSA, B=1 S=65536 Hq=64 Hkv=8 Hp=16 Hpkv=8 top_k=32 blocks, sharded by KV group"),
}
SCALE = 128 ** -0.5


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
def cpu_eager_fn(cfg, slice_cfg):
    """(callable, kind): the reference project's own eager model when its copy under oracle/_ref imports here
    ("reference"), else the oracle's line-by-line restatement of it ("port")."""
    from oracle import make_ref
    from oracle import msa_oracle as O
    models = make_ref.reference_eager()
    if models is not None:
        cls = models[1] if cfg["dense"] else models[0]
        m = cls(slice_cfg["hq"], slice_cfg["hkv"], 128, slice_cfg["hp"], slice_cfg["hpkv"], max(cfg["kb"], 1) * 128, False)
        return (lambda *t: m._attention_eager(*t)), "reference"
    if cfg["dense"]:
        return (lambda *t: O.eager_warmup(*t, SCALE)), "port"
    return (lambda *t: O.eager_sparse(*t, cfg["kb"] * 128, SCALE)), "port"


def cpu_slice_step(fn, tensors):
    """One fwd+bwd of the reference's eager algorithm on one (batch, KV group) slice."""
    from oracle import msa_oracle as O
    qp, kp, q, k, v, do = tensors
    O.eager_forward_backward(fn, (qp, kp, q, k, v), do, 1.0)


def cpu_slice(cfg, seed=0):
    """Slice geometry: one batch element, one KV head with its main and proxy heads."""
    from oracle import msa_oracle as O
    g = cfg["hq"] // cfg["hkv"]
    ppk = cfg["hp"] // cfg["hkv"]
    pkv = max(1, cfg["hpkv"] // cfg["hkv"])
    tensors = O.make_inputs(1, cfg["s"], g, 1, ppk, min(pkv, ppk), seed=seed)
    slices = cfg["b"] * cfg["hkv"]
    sl = dict(cfg, b=1, hq=g, hkv=1, hp=ppk, hpkv=min(pkv, ppk))
    return tensors, slices, flops(sl), sl


def run_cpu_baseline(cfg, steps, warmup):
    torch.set_num_threads(os.cpu_count() or 1)
    tensors, slices, f_slice, sl = cpu_slice(cfg)
    fn, kind = cpu_eager_fn(cfg, sl)
    for _ in range(warmup):
        cpu_slice_step(fn, tensors)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_slice_step(fn, tensors)
        times.append(time.perf_counter() - t0)
    t = sum(times) / len(times)
    what = "the reference's own eager model" if kind == "reference" else "fp32 eager restatement"
    return {"value": f_slice / t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"1 of {slices} (batch, KV-head group) slices of the workload per step "
                      f"(S={cfg['s']}, {cfg['hq'] // cfg['hkv']} main heads), {what}, fp32, {steps} step(s)",
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
        "config": config_of(cfg, local_problem(args.workload, 0, max(1, args.gpus))[1]),
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
# the reference's own GPU kernels beside ours (best effort: they are JIT-built at first use)
# --------------------------------------------------------------------------------------------
def ref_kernels(args):
    """Imports the reference's kernel wrappers from oracle/_ref (written by oracle/make_ref.py) and runs the three
    that need no FlashAttention backend - select_blocks (flash_msa/msa_select_cutedsl.py:481-538),
    build_reverse_index_cuda (flash_msa/reverse_index_cuda.py:139-187) and run_fused_backward
    (flash_msa/msa_backward_cutedsl.py:1083-1114) - beside fmsa_select_*, fmsa_reverse_index and fmsa_sparse_bwd on
    the same inputs, with the max-abs error of both backward kernels against the fp32 oracle.  Whatever fails to
    import, build or run is reported with its exception text instead.  Prints one JSON line."""
    import traceback
    from oracle import msa_oracle as O
    out = {"ref_kernels": {}, "shapes": []}
    refdir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(os.path.join(refdir, "flash_msa")):
        print(json.dumps({"ref_kernels": {"unavailable": "oracle/_ref is absent (run oracle/make_ref.py where the reference tree is)"}}))
        return
    sys.path.insert(0, refdir)
    dev = torch.device("cuda", 0)
    from flash_msa_b200 import ops

    def attempt(name, fn):
        try:
            return fn()
        except Exception as e:      # noqa: BLE001 - the exception text IS the result
            out["ref_kernels"][name] = {"error": f"{type(e).__name__}: {str(e)[:400]}",
                                        "where": traceback.format_exc().strip().splitlines()[-3:][0][:200]}
            return None

    def timed(fn, n=5):
        fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in ev:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in ev)

    # one attempt to import an FA4 backend under the name the reference's forward uses
    attempt("flash_attn_backend", lambda: __import__("vllm.vllm_flash_attn.cute.interface"))
    if "flash_attn_backend" not in out["ref_kernels"]:
        out["ref_kernels"]["flash_attn_backend"] = {"import": "vllm.vllm_flash_attn.cute.interface imports; not wired into the reference forward"}

    shapes = [dict(b=1, s=2048, hq=16, hkv=2, hp=4, hpkv=1, kb=4, tag="reference default (tests/test_eager_match.py)"),
              dict(WORKLOADS["c2q"], tag="quarter of c2")]
    for cfg in shapes:
        tag = cfg["tag"]
        res = {}
        qp, kp, q, k, v, do = [t.to(dev) for t in O.make_inputs(cfg["b"], cfg["s"], cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"],
                                                                seed=0, dtype=torch.bfloat16)]
        nb, kb, mpp = cfg["s"] // 128, cfg["kb"], cfg["hq"] // cfg["hp"]
        idx = ops.select_blocks(qp, kp, scale=SCALE, num_blocks=nb, top_k_blocks=kb)
        res["ours_select_ms"] = timed(lambda: ops.select_blocks(qp, kp, scale=SCALE, num_blocks=nb, top_k_blocks=kb))
        res["ours_reverse_index_ms"] = timed(lambda: ops.build_reverse_index(idx))

        def ref_select():
            from flash_msa.msa_select_cutedsl import select_blocks
            r = select_blocks(qp, kp, scale=SCALE, num_blocks=nb, top_k_blocks=kb)
            res["ref_select_ms"] = timed(lambda: select_blocks(qp, kp, scale=SCALE, num_blocks=nb, top_k_blocks=kb))
            same = (r.sort(-1).values == idx.sort(-1).values).all(-1).float().mean().item()
            res["rows_with_same_selection"] = same      # the reference rounds scores to bf16 first: ties differ
            return r
        attempt(f"select_blocks [{tag}]", ref_select)

        meta = {}

        def ref_rix():
            from flash_msa.reverse_index_cuda import build_reverse_index_cuda
            qc = 128 // mpp
            meta["tm"], meta["tq"] = build_reverse_index_cuda(idx, query_chunk=qc)
            res["ref_reverse_index_ms"] = timed(lambda: build_reverse_index_cuda(idx, query_chunk=qc))
        attempt(f"build_reverse_index_cuda [{tag}]", ref_rix)

        # backward: both kernels get the same forward results (ours) and are measured against the oracle
        rix = ops.build_reverse_index(idx)
        o, lse, lse_p = ops.attention_forward(q, k, v, qp, kp, SCALE, rix)
        gk = torch.ones((), device=dev)
        ours = ops.attention_backward(q, k, v, qp, kp, o, do, lse, lse_p, SCALE, rix, gk)
        res["ours_backward_ms"] = timed(lambda: ops.attention_backward(q, k, v, qp, kp, o, do, lse, lse_p, SCALE, rix, gk))
        names = ["dq_proxy", "dk_proxy", "dq", "dk", "dv"]
        want = None
        if cfg["s"] <= 2048:
            want = O.sparse_forward_backward(qp, kp, q, k, v, kb * 128, SCALE, do, 1.0, block_indices=idx)
            res["ours_max_abs_err"] = {n: (g_.float() - want[n]).abs().max().item() for n, g_ in zip(names, ours)}

        def ref_bwd():
            from flash_msa.msa_backward_cutedsl import run_fused_backward
            go = do.view(cfg["b"], cfg["s"], cfg["hq"], 128).transpose(1, 2).contiguous()
            om = o.view(cfg["b"], cfg["s"], cfg["hq"], 128).transpose(1, 2).contiguous()
            delta = (om.float() * go.float()).sum(-1)
            call = lambda: run_fused_backward(qp, kp, q, k, v, go, lse, lse_p, delta, meta["tm"], meta["tq"], scale=SCALE,
                                              grad_kl_scale=1.0 / (cfg["b"] * cfg["hp"] * cfg["s"]))
            grads = call()
            res["ref_backward_ms"] = timed(call)
            if want is not None:
                res["ref_max_abs_err"] = {n: (g_.float() - want[n]).abs().max().item() for n, g_ in zip(names, grads)}
        if "tm" in meta:
            attempt(f"run_fused_backward [{tag}]", ref_bwd)
        out["shapes"].append({"shape": {k_: v_ for k_, v_ in cfg.items() if k_ not in ("desc", "tag", "dense")}, "tag": tag, **res})
    print(json.dumps(out))


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
SHARDING_NOTE = "(batch, KV-head group), no collective on the kernel path"
L2_NOTE = "inputs larger than L2 (no flush needed)"


def config_of(cfg, local):
    """The `config` object of the JSON line; both arms emit the same one for the same workload."""
    return {"workload": cfg["desc"], "sharding": SHARDING_NOTE, "l2": L2_NOTE, "per_rank": local}


def local_problem(name, rank, world):
    """Per-rank problem and scaling mode of a workload: config 5 is one global problem split by KV group (strong
    scaling); every other workload is replicated, one full problem per rank (weak scaling)."""
    from flash_msa_b200.sharding import shard_workload
    cfg = dict(WORKLOADS[name])
    if name == "c5":
        return cfg, shard_workload(cfg, rank, world), "strong"
    return cfg, dict(cfg), "weak"


def bwd_traffic_bytes(workload):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary (profiles/traffic_c2q.json: a
    capture of the quarter-size case; traffic is proportional to the (batch, KV group) units processed)."""
    path = os.path.join(ROOT, "profiles", "traffic_c2q.json")
    if workload != "c2" or not os.path.exists(path):
        return None
    with open(path) as f:
        t = json.load(f)
    return float(t["scale_to_c2"]) * (float(t["dram_bytes_read"]) + float(t["dram_bytes_write"]))


class GpuContext:
    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (flash_msa_b200 has no CPU path)")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def sync_all(self):
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        if self.dist is None:
            return ms
        t = torch.tensor([ms], device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def time_workload(ctx, name, steps, warmup, with_e2e, sample_clocks, docs=0):
    """W warm-up steps, then K timed fwd+bwd steps of one workload on this rank's share of it (CUDA events on the
    launching stream, barrier + synchronize on both sides, max over ranks)."""
    import flash_msa_b200
    from flash_msa_b200 import ops
    from oracle.msa_oracle import make_inputs

    cfg, local, scaling = local_problem(name, ctx.rank, ctx.world)
    dev = ctx.dev
    fn = flash_msa_b200.flash_msa_warmup_func if cfg["dense"] else flash_msa_b200.flash_msa_func
    top_k = cfg["kb"] * 128
    cu = None
    if docs > 0:
        # packed sequences: `docs` documents of (nearly) equal length whose boundaries do not fall on block boundaries
        fn = flash_msa_b200.flash_msa_warmup_varlen_func if cfg["dense"] else flash_msa_b200.flash_msa_varlen_func
        cu = [0] + [min(local["s"], i * local["s"] // docs + 37) for i in range(1, docs)] + [local["s"]]
    host = make_inputs(local["b"], local["s"], local["hq"], local["hkv"], local["hp"], local["hpkv"], seed=ctx.rank,
                       dtype=torch.bfloat16, skew=bool(cfg.get("skew", False)))
    host = [t.pin_memory() for t in host]
    qp, kp, q, k, v, do = [t.to(dev) for t in host]
    ones = torch.ones((), device=dev)

    def step():
        leaves = [t.detach().requires_grad_(True) for t in (qp, kp, q, k, v)]
        out, kl = fn(*leaves, top_k, SCALE) if cu is None else fn(*leaves, cu, top_k, SCALE)
        torch.autograd.backward([out, kl], [do, ones])

    for _ in range(warmup):
        step()
    ctx.sync_all()
    sampler = ClockSampler(ctx.local_rank) if (sample_clocks and ctx.rank == 0) else None
    if sampler:
        sampler.start()
    torch.cuda.reset_peak_memory_stats(dev)
    ops.KERNEL_EVENTS = []
    launches0 = ops.LAUNCHES
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.sync_all()
    start.record()
    for _ in range(steps):
        step()
    end.record()
    ctx.sync_all()
    elapsed_ms = ctx.max_over_ranks(start.elapsed_time(end))
    res = {"cfg": cfg, "local": local, "scaling": scaling, "steps": steps, "ms_per_step": elapsed_ms / steps,
           "launches": ops.LAUNCHES - launches0, "clocks": sampler.stop() if sampler else None,
           "peak_mem_gib": torch.cuda.max_memory_allocated(dev) / 2 ** 30}
    events, ops.KERNEL_EVENTS = ops.KERNEL_EVENTS, None
    per_kernel = {}
    for kname, s_, e_ in events:
        per_kernel.setdefault(kname, []).append(s_.elapsed_time(e_))
    res["per_kernel"] = per_kernel
    step_total = sum(sum(v_) for v_ in per_kernel.values()) / steps
    res["kernels"] = {n: {"ms_per_step": sum(v_) / steps, "share": (sum(v_) / steps) / step_total if step_total else None}
                      for n, v_ in sorted(per_kernel.items())}

    # ---- end to end: host buffers, copies inside the timed region ----
    if with_e2e:
        # the repo's host-buffer call: pinned host tensors in, pinned host tensors out, copies and kernels
        # pipelined over (batch, KV-group) chunks on three streams (flash_msa_b200/host.py)
        from flash_msa_b200.host import HostStep
        hs = HostStep(local["b"], local["s"], local["hq"], local["hkv"], local["hp"], local["hpkv"], top_k, SCALE,
                      dense=cfg["dense"], device=dev)
        for _ in range(max(3, min(warmup, 5))):   # warm-up: pinned buffers touched, streams and clocks settled
            hs.run(*host, grad_kl=1.0)
        hs.synchronize()
        ctx.sync_all()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(2, min(steps, 5))
        allocs0 = torch.cuda.memory_stats(dev).get("num_device_alloc", 0)
        s2.record()
        for _ in range(n_e2e):
            hs.run(*host, grad_kl=1.0)
        # the step ends when the last result has reached host memory
        torch.cuda.current_stream().wait_stream(hs.s_out)
        torch.cuda.current_stream().wait_stream(hs.s_cmp)
        e2.record()
        ctx.sync_all()
        e2e_ms = ctx.max_over_ranks(s2.elapsed_time(e2))
        # cudaMalloc calls of the caching allocator inside the timed steps (each one waits for the device): 0 in a steady pipeline
        e2e_allocs = torch.cuda.memory_stats(dev).get("num_device_alloc", 0) - allocs0
        h2d, d2h = hs.bytes_per_step()
        # Copy-only floor: the same bytes as one contiguous pinned copy per tensor in each direction, both
        # directions at once, every rank at the same time.  What the host link gives whatever the kernels do.
        outs_dev = [torch.empty_like(t, device=dev) for t in hs.host_out]
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        dev_in = [qp, kp, q, k, v, do]

        def copies():
            with torch.cuda.stream(s_in):
                for d_, h_ in zip(dev_in, host):
                    d_.copy_(h_, non_blocking=True)
            with torch.cuda.stream(s_out):
                for h_, d_ in zip(hs.host_out, outs_dev):
                    h_.copy_(d_, non_blocking=True)

        copies()
        ctx.sync_all()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(3):
            copies()
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)
        c1.record()
        ctx.sync_all()
        floor_ms = ctx.max_over_ranks(c0.elapsed_time(c1)) / 3
        total_f = flops(cfg) * (ctx.world if scaling == "weak" else 1)
        res["e2e"] = {"value": total_f * n_e2e / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / n_e2e, "steps": n_e2e, "copy_floor_ms": floor_ms,
                      "device_allocs_in_timed_steps": e2e_allocs}
        del hs, outs_dev
    del qp, kp, q, k, v, do, host
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--varlen-docs", type=int, default=0,
                    help="also time the workload as a packed sequence of this many documents (document masking)")
    ap.add_argument("--no-strong-c5", action="store_true", help="skip the config-5 strong-scaling measurement of the default run")
    ap.add_argument("--micro-select", action="store_true", help="time the top-k and reverse-index kernels at config-5 size")
    ap.add_argument("--ref-kernels", action="store_true", help="try the reference's own GPU kernels beside ours (needs oracle/_ref)")
    args = ap.parse_args()
    if args.micro_select:
        micro_select(args)
        return
    if args.ref_kernels:
        ref_kernels(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 0)
    cfg = dict(WORKLOADS[args.workload])

    if args.impl == "reference":
        reference_arm(args, cfg)
        return

    ctx = GpuContext()
    main_res = time_workload(ctx, args.workload, args.steps, args.warmup, with_e2e=not args.no_e2e, sample_clocks=True)
    # Config 5 (long context, one global problem split by KV group) next to the headline: the strong-scaling curve
    # comes from running this same command at 1, 2, 4 and 8 GPUs.
    strong = None
    if args.workload == "c2" and not args.no_strong_c5 and WORKLOADS["c5"]["hkv"] % ctx.world == 0:
        strong = time_workload(ctx, "c5", max(2, min(args.steps, 5)), 2, with_e2e=False, sample_clocks=False)

    packed = None
    if args.varlen_docs > 0:
        packed = time_workload(ctx, args.workload, max(2, min(args.steps, 5)), 3, with_e2e=False, sample_clocks=False,
                               docs=args.varlen_docs)

    if ctx.rank != 0:
        if ctx.dist is not None:
            ctx.dist.destroy_process_group()
        return

    world = ctx.world
    cfg, local, scaling = main_res["cfg"], main_res["local"], main_res["scaling"]
    peaks = measured_peaks()
    total_flops = flops(cfg) * (world if scaling == "weak" else 1)
    ms_per_step = main_res["ms_per_step"]
    value = total_flops / (ms_per_step * 1e-3) / 1e12
    tokens = cfg["b"] * cfg["s"] * (world if scaling == "weak" else 1)

    # dominant kernel: the fused backward.  Algorithmic FLOPs per launch = 5 products over the
    # selected pairs of this rank's problem.
    bwd_times = main_res["per_kernel"].get("attn_bwd", [float("nan")])
    bwd_ms_step = sum(bwd_times) / main_res["steps"]     # all launches of one step (large problems run in passes)
    bwd_launches = len(bwd_times) / main_res["steps"]
    bwd_flops = flops(local) * 5.0 / 7.0
    achieved = bwd_flops / (bwd_ms_step * 1e-3) / 1e12
    traffic = bwd_traffic_bytes(args.workload) if bwd_launches == 1 else None
    roofline = {"kernel": "sparse_bwd_kernel", "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "traffic": traffic,
                "peak_source": f"{peaks['source']} (burst cuBLAS bf16)", "ms_per_launch": bwd_ms_step / bwd_launches,
                "launches_per_step": bwd_launches}

    line = {
        "metric": "sparse_attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_of(cfg, local),
        "tokens_per_s": tokens / (ms_per_step * 1e-3),
        "frac_of_peak": value / (peaks["bf16_tflops"] * world),
        "roofline": roofline, "kernels": main_res["kernels"], "clocks": main_res["clocks"],
        "gpu_launches": main_res["launches"], "peak_mem_gib": main_res["peak_mem_gib"],
    }
    if "e2e" in main_res:
        line["e2e"] = main_res["e2e"]
    if strong is not None:
        c5 = strong["cfg"]
        t5 = strong["ms_per_step"] * 1e-3
        line["strong_c5"] = {"workload": c5["desc"], "n_gpus": world, "scaling": "strong", "steps": strong["steps"],
                             "ms_per_step": strong["ms_per_step"], "tokens_per_s": c5["b"] * c5["s"] / t5,
                             "tflops": flops(c5) / t5 / 1e12, "per_rank": strong["local"], "kernels": strong["kernels"],
                             "peak_mem_gib": strong["peak_mem_gib"]}
    if packed is not None:
        line["varlen"] = {"docs": args.varlen_docs, "steps": packed["steps"], "ms_per_step": packed["ms_per_step"],
                          "kernels": packed["kernels"],
                          "note": "same tensors as a packed sequence; fewer visible (query, key) pairs, so no TFLOP/s figure"}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = {k_: v_ for k_, v_ in run_cpu_baseline(cfg, 1, 1).items() if k_ not in ("s_per_slice", "slices")}
    print(json.dumps(line))
    if ctx.dist is not None:
        ctx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
