"""Helpers shared by the GPU parity tests."""
import torch

from oracle import msa_oracle as O

SCALE = 128 ** -0.5


def bf16_inputs(cfg, device="cuda", layout="bhsd", skew=False, dtype=torch.bfloat16):
    """Seeded inputs, rounded to bf16 (or to `dtype`).  layout "bshd" returns (B,H,S,D) views of (B,S,H,D)
    storage, the layout the reference's callers pass (flash_msa/tests/testing_model.py:173-185)."""
    ts = O.make_inputs(cfg["b"], cfg["s"], cfg["hq"], cfg["hkv"], cfg["hp"], cfg["hpkv"], seed=cfg.get("seed", 0),
                       dtype=dtype, device=device, skew=skew)
    qp, kp, q, k, v, do = ts
    if layout == "bshd":
        qp, kp, q, k, v = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (qp, kp, q, k, v))
    return qp, kp, q, k, v, do


def max_err(a, ref):
    return (a.double() - ref.double()).abs().max().item()


def yardstick_check(name, got, ref32, ref16, floor):
    """Error of the kernel against the fp32 oracle must stay within twice the error of the
    reference's own bf16 eager arithmetic against the same oracle (plus a small absolute floor
    for tensors whose bf16 error happens to be tiny)."""
    e_k = max_err(got, ref32)
    e_y = max_err(ref16, ref32)
    assert e_k <= 2.0 * e_y + floor, f"{name}: kernel err {e_k:.3e} vs yardstick {e_y:.3e}"
    return e_k, e_y


def yardstick_ratio(got, ref32, ref16):
    """Kernel error divided by the yardstick error plus 1e-3 of the largest reference element (rows whose
    gradient is exactly zero have a zero yardstick error).  For reporting."""
    return max_err(got, ref32) / (max_err(ref16, ref32) + 1e-3 * ref32.abs().max().item() + 1e-6)


def kernel_selection(q_proxy, k_proxy, kb):
    """The block selection the forward makes for these inputs (the select kernels are deterministic, so
    calling them again reproduces what `flash_msa_func` used)."""
    from flash_msa_b200 import ops
    return ops.select_blocks(q_proxy, k_proxy, scale=SCALE, num_blocks=q_proxy.shape[2] // 128, top_k_blocks=kb)


_REPORT = {}


def report(section, values):
    """Collects parity figures (error / yardstick ratios, near-tie and flip counts) of the GPU tests into one
    JSON file: $FMSA_PARITY_REPORT, or parity_report.json in the scratch output folder under the repository root."""
    import json
    import os
    _REPORT[section] = values
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.environ.get("FMSA_PARITY_REPORT") or os.path.join(root, "gpurun_out", "parity_report.json")
    try:
        os.makedirs(os.path.dirname(path), exist_ok=True)
        old = {}
        if os.path.exists(path):
            with open(path) as f:
                old = json.load(f)
        old.update(_REPORT)
        with open(path, "w") as f:
            json.dump(old, f, indent=1, sort_keys=True)
    except OSError:
        pass
