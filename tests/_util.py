"""Shared helpers of the parity tests."""

import numpy as np
import torch

# Tolerance of every floating-point parity test (GEMV / GEMM / attention outputs):
# element-wise relative error against the float64 oracle result rounded to the
# output type; |ref| is floored at 1% of the RMS of ref so that outputs which
# cancel to ~0 do not divide by nothing.
MAX_REL = 1e-2
MEAN_REL = 1e-3


def rel_errors(got: np.ndarray, ref64: np.ndarray, out_dtype: torch.dtype):
    ref = torch.from_numpy(np.asarray(ref64, dtype=np.float64)).to(out_dtype).double().numpy()
    got = np.asarray(got, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref * ref))) or 1.0
    den = np.maximum(np.abs(ref), 1e-2 * rms)
    err = np.abs(got - ref) / den
    return float(err.max()), float(err.mean())


def assert_close(got, ref64, out_dtype, what=""):
    mx, mean = rel_errors(got, ref64, out_dtype)
    assert mx <= MAX_REL and mean <= MEAN_REL, f"{what}: max rel {mx:.3e} mean rel {mean:.3e}"


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.dtype in (torch.float16, torch.bfloat16) \
        else t.detach().cpu().numpy()


def same_bits_f32(a: np.ndarray, b: np.ndarray) -> bool:
    return a.dtype == b.dtype == np.float32 and np.array_equal(a.view(np.uint32), b.view(np.uint32))


# Token count from which linears take the tensor-core GEMM (GEMM_TC_MIN_M in csrc/linear.cuh), whose
# definition rounds the decoded weight to the activation type once, as the reference's tiled GEMM does.
GEMM_MIN_TOKENS = 28
