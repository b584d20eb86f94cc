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


# ---- device staging (GPU tests) ----------------------------------------------------------

def stage_layer(experts: dict, num_experts: int, hidden: int, inter: int, encoding: str, device):
    """Concatenate canonical bytes of the given experts {e: (gate, up, down) EncodedMatrix}
    into a DeviceLayer; experts not listed stay zero (scales 1)."""
    from uma_qmoe_b200.formats import row_bytes
    from uma_qmoe_b200.ops import DeviceLayer

    q = encoding != "bf16_le"
    gu = np.zeros((num_experts, inter * row_bytes(encoding, hidden)), np.uint8)
    up = np.zeros_like(gu)
    dn = np.zeros((num_experts, hidden * row_bytes(encoding, inter)), np.uint8)
    gs = np.ones((num_experts, inter * hidden // 128), np.float32)
    us = np.ones_like(gs)
    ds = np.ones((num_experts, hidden * inter // 128), np.float32)
    for e, (g, u, d) in experts.items():
        gu[e] = np.frombuffer(g.data.tobytes(), np.uint8)
        up[e] = np.frombuffer(u.data.tobytes(), np.uint8)
        dn[e] = np.frombuffer(d.data.tobytes(), np.uint8)
        if q:
            gs[e], us[e], ds[e] = g.scales, u.scales, d.scales
    dev = lambda a: torch.from_numpy(a).to(device)
    return DeviceLayer(encoding, num_experts, hidden, inter, dev(gu), dev(up), dev(dn),
                       dev(gs) if q else None, dev(us) if q else None, dev(ds) if q else None)


def assert_parity(actual: torch.Tensor, expected: torch.Tensor, max_abs: float = 2e-2, cosine: float = 0.9999):
    """The activation tolerance of the operator contract: max-abs <= 2e-2 and cosine >= 0.9999
    against the CPU correctness path."""
    m = orc.compare(actual, expected)
    assert m["max_abs"] <= max_abs and m["cosine"] >= cosine, m
    return m
