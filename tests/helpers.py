"""Shared helpers for the parity tests."""

from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

DT_TAG = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}
TAG_DT = {v: k for k, v in DT_TAG.items()}


def load_golden(name: str) -> dict:
    with np.load(os.path.join(GOLDEN_DIR, name)) as data:
        return {k: data[k] for k in data.files}


def to_np(t: torch.Tensor) -> np.ndarray:
    """Tensor -> NumPy; 16-bit floats are widened to float32 (exact)."""

    t = t.detach().cpu()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.float().numpy().copy()
    return t.numpy().copy()
