"""Deterministic inputs of the golden vectors (same function as tests/golden/make_golden.py:inputs)."""

from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def inputs(seed: int, T: int, H: int, I: int, E: int, glu: bool = True) -> dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    f = lambda *s: rng.standard_normal(s, dtype=np.float32)
    return {
        "x": f(T, H),
        "gate": f(E, H) * np.float32(0.02),
        "w_fc": f(E, (2 if glu else 1) * I, H) * np.float32(0.02),
        "w_proj": f(E, H, I) * np.float32(0.02),
        "grad_y": f(T, H),
    }


def load(name: str) -> tuple[dict[str, torch.Tensor], dict[str, torch.Tensor], dict[str, int]]:
    """Returns (inputs, reference outputs, meta) of one golden file as torch tensors."""
    rec = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    seed, T, H, I, E, k, glu = (int(v) for v in rec["meta"])
    inp = {key: torch.from_numpy(val) for key, val in inputs(seed, T, H, I, E, bool(glu)).items()}
    out = {key: torch.from_numpy(np.asarray(rec[key])) for key in rec.files if key != "meta"}
    return inp, out, dict(seed=seed, T=T, H=H, I=I, E=E, k=k, glu=glu)


def sample(t: torch.Tensor, step: int = 37) -> torch.Tensor:
    return t.reshape(-1)[::step]
