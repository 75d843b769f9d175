"""Make the unmodified reference available to the checker and to the benchmark's reference arm.

TEST / BENCHMARK INFRASTRUCTURE - nothing in the shipped package imports what this script writes.

    python oracle/build_ref.py [/path/to/reference/checkout]

Two outputs, both ignored by git (they are the reference's own code, not this project's):

  baseline/_ref/          ``pip install --target`` of the reference's ``ommx_gpu_serve`` package
                          (pure Python + Triton): its packer, its fp32 oracle and its Triton decode
                          kernels, run on the GPU by tests/test_triton_reference_gpu.py and timed
                          by bench.py beside this project's kernels.
  oracle/_ref/ommx_fakequant/quant_function.py
                          the reference's CPU fake quantizer (a single torch-only module that
                          belongs to no installable package), timed by ``bench.py --impl
                          reference`` as the CPU baseline.

The checkout is read where it lies; the install runs from a scratch copy because a wheel build
writes into its source tree.  When the checkout is absent the script leaves what is already
there alone and says so.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASELINE_REF = os.path.join(ROOT, "baseline", "_ref")
ORACLE_REF = os.path.join(ROOT, "oracle", "_ref")
# where a reference checkout is looked for when none is named: OMMX_REFERENCE_CHECKOUT, else "reference" beside this repository
DEFAULT_CHECKOUT = os.environ.get("OMMX_REFERENCE_CHECKOUT") or os.path.join(os.path.dirname(ROOT), "reference")


def have_triton_reference() -> bool:
    return os.path.isfile(os.path.join(BASELINE_REF, "ommx_gpu_serve", "attention", "paged_decode.py"))


def have_fakequant_reference() -> bool:
    return os.path.isfile(os.path.join(ORACLE_REF, "ommx_fakequant", "quant_function.py"))


def build_ref(checkout: str = "", force: bool = False) -> dict:
    """Install / copy the reference pieces; returns {'triton': bool, 'fakequant': bool, 'log': str}."""
    log = []
    checkout = checkout or DEFAULT_CHECKOUT
    pkg_src = os.path.join(checkout, "ommx_gpu_serve")
    if os.path.isdir(pkg_src) and (force or not have_triton_reference()):
        with tempfile.TemporaryDirectory() as tmp:
            src = os.path.join(tmp, "ommx_gpu_serve")
            shutil.copytree(pkg_src, src, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
            if os.path.isdir(BASELINE_REF):
                shutil.rmtree(BASELINE_REF)
            cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                   "--find-links", "/opt/wheelhouse", "--target", BASELINE_REF, src]
            res = subprocess.run(cmd, capture_output=True, text=True)
            log.append("pip install ommx_gpu_serve -> baseline/_ref: " +
                       ("ok" if res.returncode == 0 else "FAILED\n" + res.stdout[-2000:] + res.stderr[-2000:]))
    # The package also ships the C++/CUDA sources of the reference's weight-linear kernels as data files.  Nothing
    # on the attention path loads them, and they name TMA loads with cluster multicast, which this project keeps out
    # of everything that ships with code run on two or more GPUs: drop them.
    csrc = os.path.join(BASELINE_REF, "ommx_gpu_serve", "csrc")
    if os.path.isdir(csrc):
        shutil.rmtree(csrc)
        log.append("baseline/_ref/ommx_gpu_serve/csrc (weight-linear kernel sources, unused here): removed")
    elif not os.path.isdir(pkg_src):
        log.append(f"{pkg_src} not present: baseline/_ref left as it is")
    fq_src = os.path.join(checkout, "ommx_fakequant", "quant_function.py")
    if os.path.isfile(fq_src) and (force or not have_fakequant_reference()):
        dst = os.path.join(ORACLE_REF, "ommx_fakequant")
        os.makedirs(dst, exist_ok=True)
        shutil.copyfile(fq_src, os.path.join(dst, "quant_function.py"))
        log.append("ommx_fakequant/quant_function.py -> oracle/_ref: ok")
    elif not os.path.isfile(fq_src):
        log.append(f"{fq_src} not present: oracle/_ref left as it is")
    return {"triton": have_triton_reference(), "fakequant": have_fakequant_reference(), "log": "\n".join(log)}


if __name__ == "__main__":
    out = build_ref(next((a for a in sys.argv[1:] if not a.startswith("--")), ""), force="--force" in sys.argv)
    print(out["log"])
    print({k: v for k, v in out.items() if k != "log"})
