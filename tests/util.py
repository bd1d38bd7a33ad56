"""Shared helpers of the parity tests: host arrays <-> device tensors and the
two error measures the tolerances are stated in."""
import numpy as np
import torch

from oracle import svod_oracle as O

TORCH_DTYPE = {O.BF16: torch.bfloat16, O.F16: torch.float16, O.F32: torch.float32}


def dev(x, dtype):
    """A host array of values already rounded to `dtype` -> CUDA tensor (exact)."""
    t = torch.from_numpy(np.ascontiguousarray(np.asarray(x, dtype=np.float32)))
    return t.to(TORCH_DTYPE[dtype]).cuda()


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def max_abs(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    both_inf = np.isinf(got) & np.isinf(want) & (np.sign(got) == np.sign(want))
    d = np.where(both_inf, 0.0, np.abs(got - want))
    return float(np.nanmax(d)) if d.size else 0.0


def mean_rel(got, want):
    """mean|got - want| / mean|want|."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    denom = float(np.mean(np.abs(want)))
    return float(np.mean(np.abs(got - want))) / (denom if denom > 0 else 1.0)


def rel_close(got, want, tol):
    """The reference's `assert_rel_close`: |got - want| <= tol * max(|want|, 1)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return bool(np.all(np.abs(got - want) <= tol * np.maximum(np.abs(want), 1.0)))


def normal(rng, shape, sigma, dtype):
    """Seeded N(0, sigma) values rounded to `dtype` (float64 array)."""
    return O.round_to(dtype, rng.standard_normal(shape) * sigma)
