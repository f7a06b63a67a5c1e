"""Generate the golden vectors under tests/golden/ from the reference's own eager model.

Run in a container that has the reference tree:

    REFERENCE_ROOT=/path/to/flash-msa python tests/golden/make_golden.py

It imports ``flash_msa.tests.testing_model.Model`` and
``flash_msa.tests.testing_model_warmup.WarmupModel`` from that tree (CPU, fp32), calls their
``_attention_eager`` on seeded inputs, differentiates ``sum(out*dO) + kl`` with autograd and
stores the results.  Inputs are regenerated from the seed by ``oracle.msa_oracle.make_inputs``;
a checksum of the inputs is stored so a drifting generator is detected.

Files written:
  sparse_small.npz / warmup_small.npz   full tensors, B=1 S=384 Hq=4 Hkv=1 Hp=2 Hpkv=1 top_k=256
  c1_summary.json                       BASELINE config 1 (B=1 S=1024 Hq=8 Hkv=2 Hp=2 Hpkv=2
                                        top_k=512): per-tensor sums, norms and sampled values
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
if "REFERENCE_ROOT" not in os.environ:
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference project (the directory that holds flash_msa/)")
sys.path.insert(0, os.environ["REFERENCE_ROOT"])

from flash_msa.tests.testing_model import Model                    # noqa: E402
from flash_msa.tests.testing_model_warmup import WarmupModel       # noqa: E402
from oracle import msa_oracle as O                                 # noqa: E402

NAMES = ["dq_proxy", "dk_proxy", "dq", "dk", "dv"]
SMALL = dict(b=1, s=384, hq=4, hkv=1, hp=2, hpkv=1, kb=2, seed=1)
C1 = dict(b=1, s=1024, hq=8, hkv=2, hp=2, hpkv=2, kb=4, seed=0)


def input_checksum(tensors):
    return [float(t.double().sum()) for t in tensors]


def run_reference(cfg, warmup):
    qp, kp, q, k, v, do = O.make_inputs(cfg["b"], cfg["s"], cfg["hq"], cfg["hkv"], cfg["hp"],
                                        cfg["hpkv"], seed=cfg["seed"])
    cls = WarmupModel if warmup else Model
    m = cls(cfg["hq"], cfg["hkv"], 128, cfg["hp"], cfg["hpkv"], cfg["kb"] * 128, False)
    out, kl, grads = O.eager_forward_backward(lambda *t: m._attention_eager(*t),
                                              (qp, kp, q, k, v), do, 1.0)
    res = {"out": out, "kl": kl}
    res.update(dict(zip(NAMES, grads)))
    return (qp, kp, q, k, v, do), res


def sample_index(numel, n=64):
    rng = np.random.RandomState(1234)
    return rng.randint(0, numel, size=n)


def summarise(res):
    s = {}
    for name, t in res.items():
        t = t.double().reshape(-1)
        idx = sample_index(t.numel()) if t.numel() > 1 else np.zeros(1, dtype=np.int64)
        s[name] = {
            "sum": float(t.sum()),
            "abs_sum": float(t.abs().sum()),
            "l2": float(t.pow(2).sum().sqrt()),
            "sample_idx": [int(i) for i in idx],
            "sample": [float(t[int(i)]) for i in idx],
        }
    return s


def main():
    torch.set_num_threads(os.cpu_count())
    for warmup, fname in ((False, "sparse_small.npz"), (True, "warmup_small.npz")):
        ins, res = run_reference(SMALL, warmup)
        payload = {k: v.numpy().astype(np.float32) for k, v in res.items()}
        payload["input_checksum"] = np.array(input_checksum(ins))
        payload["config"] = np.array(json.dumps(SMALL))
        np.savez_compressed(os.path.join(HERE, fname), **payload)
        print("wrote", fname)
    summary = {"config": C1}
    for warmup, key in ((False, "sparse"), (True, "warmup")):
        ins, res = run_reference(C1, warmup)
        summary[key] = summarise(res)
        summary["input_checksum"] = input_checksum(ins)
    with open(os.path.join(HERE, "c1_summary.json"), "w") as f:
        json.dump(summary, f, indent=1)
    print("wrote c1_summary.json")


if __name__ == "__main__":
    main()
