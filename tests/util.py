"""Shared helpers of the GPU parity tests: seeded inputs, bf16 views, error measures."""
import numpy as np

TOL_F32 = 1e-5    # relative Frobenius, strict f32 path
TOL_TF32 = 5e-3   # relative Frobenius, TF32 tensor path
TOL_BF16 = 2e-2   # relative Frobenius, bf16 tensor path


def rel_fro(got, want) -> float:
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    denom = np.linalg.norm(want.ravel())
    return float(np.linalg.norm((got - want).ravel()) / (denom if denom > 0 else 1.0))


def close_like_parity_zig(want, got, tolerance=2e-4) -> bool:
    """tests/parity.zig:10-18: abs(w - g) <= tolerance * max(1, abs(w)) for every element."""
    want = np.asarray(want, np.float64)
    got = np.asarray(got, np.float64)
    return bool(np.all(np.abs(want - got) <= tolerance * np.maximum(1.0, np.abs(want))))


def seeded(seed, *shape, kind="normal"):
    rng = np.random.default_rng(seed)
    if kind == "normal":
        return rng.standard_normal(shape, dtype=np.float32)
    if kind == "uniform_half":   # U(-0.5, 0.5), tests/parity.zig:66-67
        return (rng.random(shape, dtype=np.float32) - np.float32(0.5)).astype(np.float32)
    if kind == "unit":           # U[0, 1)
        return rng.random(shape, dtype=np.float32)
    raise ValueError(kind)


def to_dev(arr, bf16=False):
    """numpy f32 -> CUDA tensor; with bf16=True the values are RNE-rounded to bfloat16 storage."""
    import torch

    t = torch.from_numpy(np.ascontiguousarray(arr)).cuda()
    return t.to(torch.bfloat16) if bf16 else t


def to_host(t):
    import torch

    return t.detach().to(torch.float32).cpu().numpy()
