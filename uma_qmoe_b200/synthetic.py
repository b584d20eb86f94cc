"""Seeded synthetic inputs with the shapes and value distributions of the two
fixed models (OLMoE-1B-7B and Qwen1.5-MoE-A2.7B).

No checkpoint, tokenizer or dataset is involved: expert and router weights are
N(0, 0.02) rounded to BF16, activations are N(0, 1) rounded to BF16.  numpy's
PCG64 stream is used (not torch's) so the same seed gives the same bytes on any
host; the golden fixtures store SHA-256 digests of what these functions return.

The frozen shapes follow ``src/uma_qmoe/fixed_models.py:32-55`` of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch


@dataclass(frozen=True)
class ModelShape:
    name: str
    hidden: int
    intermediate: int
    experts: int
    top_k: int
    layers: int
    shared_intermediate: int = 0   # Qwen shared expert; 0 = none
    qwen: bool = False


OLMOE = ModelShape("olmoe", 2048, 1024, 64, 8, 16)
QWEN = ModelShape("qwen", 2048, 1408, 60, 4, 24, shared_intermediate=5632, qwen=True)


def _bf16_round(a: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even BF16 -> float32 (values exactly representable in BF16)."""
    w = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = np.uint32(0x7FFF) + ((w >> 16) & 1)
    return (((w + r) >> 16) << 16).astype(np.uint32).view(np.float32)


def normal_bf16(seed: tuple[int, ...], shape: tuple[int, ...], std: float) -> np.ndarray:
    rng = np.random.default_rng(list(seed))
    return _bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def expert_weights(seed: int, layer: int, expert: int, shape: ModelShape
                   ) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(gate [I,H], up [I,H], down [H,I]) float32 arrays holding BF16 values."""
    gate = normal_bf16((seed, layer, expert, 0), (shape.intermediate, shape.hidden), 0.02)
    up = normal_bf16((seed, layer, expert, 1), (shape.intermediate, shape.hidden), 0.02)
    down = normal_bf16((seed, layer, expert, 2), (shape.hidden, shape.intermediate), 0.02)
    return gate, up, down


def router_weight(seed: int, layer: int, shape: ModelShape, skew: float = 0.0) -> torch.Tensor:
    """[E, H] BF16.  ``skew`` > 0 multiplies row e by exp(skew * z_e), z_e ~ N(0,1):
    plain N(0, 0.02) rows give nearly uniform expert loads, the scaled rows give
    the skewed loads (a few hot experts, some with no token) of a real prefill."""
    w = normal_bf16((seed, layer, 1000), (shape.experts, shape.hidden), 0.02)
    if skew:
        z = np.random.default_rng([seed, layer, 1001]).standard_normal(shape.experts)
        w = _bf16_round(w * np.exp(skew * z).astype(np.float32)[:, None])
    return torch.from_numpy(w).to(torch.bfloat16)


def activations(seed: int, tokens: int, hidden: int = 2048) -> torch.Tensor:
    """[tokens, hidden] BF16 N(0, 1)."""
    return torch.from_numpy(normal_bf16((seed, 2000), (tokens, hidden), 1.0)).to(torch.bfloat16)


def shared_expert_weights(seed: int, layer: int, shape: ModelShape
                          ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Qwen shared expert (gate [S,H], up [S,H], down [H,S]) and its sigmoid
    gate [1,H], all BF16."""
    s = shape.shared_intermediate
    mk = lambda tag, shp: torch.from_numpy(normal_bf16((seed, layer, tag), shp, 0.02)).to(torch.bfloat16)
    return (mk(3000, (s, shape.hidden)), mk(3001, (s, shape.hidden)),
            mk(3002, (shape.hidden, s)), mk(3003, (1, shape.hidden)))


def skewed_routes(seed: int, tokens: int, shape: ModelShape, pool: int,
                  ) -> tuple[torch.Tensor, torch.Tensor]:
    """Distinct top-k expert ids per token drawn from the first ``pool`` experts
    with Zipf-like popularity (so that some experts get no token), and positive
    float32 weights that sum to at most one per token."""
    rng = np.random.default_rng([seed, 4000])
    p = 1.0 / np.arange(1, pool + 1) ** 1.2
    p /= p.sum()
    idx = np.stack([rng.choice(pool, size=shape.top_k, replace=False, p=p) for _ in range(tokens)])
    w = rng.random((tokens, shape.top_k), dtype=np.float32) + np.float32(0.05)
    w = (w / w.sum(axis=1, keepdims=True) * np.float32(0.9)).astype(np.float32)
    return torch.from_numpy(idx.astype(np.int64)), torch.from_numpy(w)
