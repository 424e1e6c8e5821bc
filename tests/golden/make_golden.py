"""Generates tests/golden/gemm_tn_golden.npz from the REFERENCE's own check.

Run in the build container, where the reference tree is mounted:
    python tests/golden/make_golden.py --reference <checkout of the reference>
The fixtures travel with the repo; nothing under tests/ reads the reference tree at run time.

What is taken from the reference (kernels/tests/gemm_test.py):
  * the ground-truth expression  torch.matmul(A.float(), B.float().T)  (:36), evaluated here on
    CPU tensors instead of CUDA tensors (the file's kernel cannot run on this hardware);
  * ``measure_error_stats`` (:4-11), imported from the file itself, applied to the ideally
    rounded result so the fixture also records what the reference's check reports for a
    perfect kernel (max / mean absolute error, and that its allclose assertion passes).
The module's top-level ``from gemm_kernels import gemm_tn_test`` is satisfied with an empty
stand-in module, because the reference's extension is Hopper-only and not built here.

Inputs come from oracle.make_inputs / make_ternary_inputs (seeded CPU generators), and are
stored in the fixture as raw 16-bit patterns, so the tests do not depend on the generator
reproducing them (a digest of the 1024^3 operands checks that it still does).
"""
from __future__ import annotations

import argparse
import contextlib
import hashlib
import os
import importlib.util
import io
import sys
import types
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))
from oracle import oracle  # noqa: E402

SMALL_CASES = [
    # name, M, N, K, seed, dtype, kind
    ("small_bf16", 128, 256, 64, 11, torch.bfloat16, "normal"),
    ("ragged_bf16", 100, 264, 72, 12, torch.bfloat16, "normal"),
    ("small_fp16", 256, 128, 192, 13, torch.float16, "normal"),
    ("ternary_bf16", 128, 256, 256, 14, torch.bfloat16, "ternary"),
    ("ternary_fp16", 64, 72, 128, 15, torch.float16, "ternary"),
]
CFG1_ROWS = [0, 1, 127, 128, 255, 256, 511, 777, 1023]


def load_reference_check(ref_root: Path):
    stub = types.ModuleType("gemm_kernels")
    stub.gemm_tn_test = None
    sys.modules.setdefault("gemm_kernels", stub)
    path = ref_root / "kernels" / "tests" / "gemm_test.py"
    spec = importlib.util.spec_from_file_location("reference_gemm_test", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.measure_error_stats


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(bits(t).tobytes()).hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("REFERENCE_ROOT"), required="REFERENCE_ROOT" not in os.environ,
                    help="root of the reference checkout (or set REFERENCE_ROOT)")
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent / "gemm_tn_golden.npz"))
    args = ap.parse_args()
    measure_error_stats = load_reference_check(Path(args.reference))
    torch.set_num_threads(1)  # one summation order, whatever machine regenerates the file

    out: dict[str, np.ndarray] = {}
    names = []
    for name, M, N, K, seed, dtype, kind in SMALL_CASES:
        A, B = (oracle.make_ternary_inputs if kind == "ternary" else oracle.make_inputs)(M, N, K, seed, dtype)
        C_ref = torch.matmul(A.float(), B.float().T)           # kernels/tests/gemm_test.py:36
        ideal = C_ref.to(dtype)
        with contextlib.redirect_stdout(io.StringIO()):
            max_err, avg_err = measure_error_stats(ideal.float(), C_ref)   # asserts allclose
        names.append(name)
        out[f"{name}/A"] = bits(A)
        out[f"{name}/B"] = bits(B)
        out[f"{name}/C_ref"] = C_ref.numpy()
        out[f"{name}/meta"] = np.array([M, N, K, seed, oracle.DTYPE_CODE[dtype], int(kind == "ternary")], dtype=np.int64)
        out[f"{name}/ideal_err"] = np.array([max_err, avg_err], dtype=np.float64)

    # Benchmark configuration 1: 1024^3, seed 0, bf16.  Sampled rows of the ground truth + operand digests.
    A, B = oracle.make_inputs(1024, 1024, 1024, 0, torch.bfloat16)
    C_ref = torch.matmul(A.float(), B.float().T)
    with contextlib.redirect_stdout(io.StringIO()):
        max_err, avg_err = measure_error_stats(C_ref.to(torch.bfloat16).float(), C_ref)
    out["cfg1/rows"] = np.array(CFG1_ROWS, dtype=np.int64)
    out["cfg1/C_ref_rows"] = C_ref[CFG1_ROWS].numpy()
    out["cfg1/ideal_err"] = np.array([max_err, avg_err], dtype=np.float64)
    out["cfg1/absmax"] = np.array([C_ref.abs().max().item()], dtype=np.float64)
    out["cfg1/digests"] = np.array([digest(A), digest(B)])
    out["names"] = np.array(names)
    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(names)} small cases + cfg1 rows")


if __name__ == "__main__":
    main()
