"""Makes the reference project's own eager model importable next to the oracle, for timing and checking only.

    python oracle/make_ref.py [REFERENCE_ROOT]        (default: $REFERENCE_ROOT, else the build machine's reference checkout)

Copies the reference's ``flash_msa`` Python package (the eager models live in ``flash_msa/tests/testing_model.py``
and ``testing_model_warmup.py``; they import the package itself) into ``oracle/_ref/``, which is excluded from
version control.  Nothing under ``oracle/_ref`` is imported by the library; ``bench.py`` uses it as the CPU baseline
(``cpu_baseline.kind = "reference"``) and for the attempt to run the reference's GPU kernels, and falls back to
the oracle's restatement when the directory is absent.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make_ref(reference_root=None) -> bool:
    root = reference_root or os.environ.get("REFERENCE_ROOT") or "/root/reference"
    src = os.path.join(root, "flash_msa")
    if not os.path.isdir(src):
        return False
    dst = os.path.join(DEST, "flash_msa")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", ".DS_Store"))
    return True


def reference_eager():
    """(Model, WarmupModel) of the reference's eager implementation, or None when oracle/_ref is absent or does not
    import on this machine."""
    if not os.path.isdir(os.path.join(DEST, "flash_msa")):
        return None
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    try:
        from flash_msa.tests.testing_model import Model
        from flash_msa.tests.testing_model_warmup import WarmupModel
        return Model, WarmupModel
    except Exception:
        return None


def reference_kernels():
    """The reference's GPU kernel wrappers that need no FlashAttention backend, as a dict
    {"select_blocks", "build_reverse_index_cuda", "run_fused_backward"}, or (None, reason)."""
    if not os.path.isdir(os.path.join(DEST, "flash_msa")):
        return None, "oracle/_ref is absent"
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    try:
        from flash_msa.msa_backward_cutedsl import run_fused_backward
        from flash_msa.msa_select_cutedsl import select_blocks
        from flash_msa.reverse_index_cuda import build_reverse_index_cuda
    except Exception as e:      # noqa: BLE001
        return None, f"{type(e).__name__}: {e}"
    return {"select_blocks": select_blocks, "build_reverse_index_cuda": build_reverse_index_cuda,
            "run_fused_backward": run_fused_backward}, ""


if __name__ == "__main__":
    ok = make_ref(sys.argv[1] if len(sys.argv) > 1 else None)
    print("oracle/_ref ready" if ok else "reference tree not found; oracle/_ref not written")
