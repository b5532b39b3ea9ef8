"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import lq_oracle as O


def seeded(shape, seed, std=1.0):
    """Seeded N(0, std) f32 array (torch generator, the goldens' convention)."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * std).numpy()


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype)


def host(t):
    return t.detach().to("cpu", torch.float32).numpy()


def bf16_round(a):
    """f32 array rounded to bf16 and back (what a bf16 tensor holds)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


def reldev(ours, ref):
    return O.rel_deviation(np.asarray(ours, np.float32), np.asarray(ref, np.float32))
