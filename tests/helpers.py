"""Shared pieces of the parity tests."""
import glob
import os

import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_cases():
    return sorted(glob.glob(os.path.join(GOLDEN_DIR, "golden_*.pt")))


def load_golden(path):
    return torch.load(path, map_location="cpu")


NAMES = ("O", "dQ", "dK", "dV", "d_pair_bias")

# Acceptance of the reference's own test (test.py:69-80): allclose(atol=1e-2, rtol=1e-2 for
# bf16, 0 for fp16) against the same-dtype naive path.
def reference_allclose(x, ref, dtype):
    rtol = 0.0 if dtype == torch.float16 else 1e-2
    return torch.allclose(ref.float().cpu(), x.float().cpu(), atol=1e-2, rtol=rtol)


# Maximum relative error (max|x-ref| / max|ref|) allowed against the fp32-upcast oracle.
REL_TOL = {torch.float32: 2e-5, torch.bfloat16: 1e-2, torch.float16: 1e-2}
