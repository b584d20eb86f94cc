"""Helpers shared by the CPU and GPU tests: regenerate the seeded weights a
golden fixture was made from and present them to the oracle."""

from __future__ import annotations

import hashlib
from functools import lru_cache

import numpy as np
import torch

from oracle import moe_oracle as orc
from uma_qmoe_b200 import synthetic as syn

SEED = 20260917


def bits_to_bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().astype(np.uint16)


def sha(*chunks: bytes) -> str:
    h = hashlib.sha256()
    for c in chunks:
        h.update(c)
    return h.hexdigest()


@lru_cache(maxsize=256)
def encoded_expert(seed: int, layer: int, expert: int, model: str, encoding: str):
    shape = syn.OLMOE if model == "olmoe" else syn.QWEN
    g, u, d = syn.expert_weights(seed, layer, expert, shape)
    return tuple(orc.encode_matrix(m, encoding) for m in (g, u, d))


def expert_source(seed: int, layer: int, model: str, encoding: str):
    return lambda e: encoded_expert(seed, layer, e, model, encoding)


def ulp_bf16(x: torch.Tensor) -> torch.Tensor:
    """Size of one BF16 ulp at |x| (float32)."""
    a = x.float().abs().clamp_min(2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(a)) - 7)
