"""Shared helpers of the test-suite: seeded synthetic inputs and parity checks."""
import os

import numpy as np
import torch

from oracle import hqmq_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make_kv(kind: str, shape, seed: int, dtype=torch.float32) -> torch.Tensor:
    """Synthetic K/V of the value distributions the benchmark configurations name."""
    g = torch.Generator().manual_seed(seed)
    B, H, T, d = shape
    x = torch.randn(B, H, T, d, generator=g)
    if kind == "hot":            # 4 fixed channels per head scaled x8
        for h in range(H):
            ch = torch.randperm(d, generator=g)[:4]
            x[:, h, :, ch] *= 8.0
    elif kind == "spiky":        # 0.5 % of chunks scaled x20
        m = torch.rand(B, H, T, d // 4, generator=g) < 0.005
        x = (x.view(B, H, T, d // 4, 4) * torch.where(m, 20.0, 1.0).unsqueeze(-1)).reshape(B, H, T, d)
    elif kind == "student":      # 2 channels per head ~ Student-t(2) x100
        for h in range(H):
            ch = torch.randperm(d, generator=g)[:2]
            z = torch.randn(B, T, 2, generator=g)
            chi = (torch.randn(B, T, 2, generator=g) ** 2 + torch.randn(B, T, 2, generator=g) ** 2) / 2
            x[:, h, :, ch] = 100.0 * z / chi.sqrt()
    elif kind != "randn":
        raise ValueError(kind)
    return x.to(dtype)


def classify_idx(idx_gpu: torch.Tensor, enc: dict, tol: float = 1e-6):
    """Index mismatches against the oracle split into allowed near-ties (oracle top-2 gap < tol)
    and real errors.  Returns (n_mismatch, n_bad)."""
    mism = idx_gpu.cpu().to(torch.int32) != enc["idx"]
    n_mis = int(mism.sum())
    n_bad = int((mism & (enc["gap"] >= tol)).sum())
    return n_mis, n_bad


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm().clamp(min=1e-30))


def load_npz(name):
    return np.load(os.path.join(GOLDEN, name))
