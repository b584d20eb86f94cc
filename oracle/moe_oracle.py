"""CPU oracle for the routed-expert MoE operator path.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy + CPU torch, the algorithm of the UMA-QMoE
reference for the one path this repository accelerates: the weight codecs
(canonical Q4, symmetric Q8, BF16), the Hugging Face top-k router that feeds the
operator, the CPU correctness implementation of ``uma_qmoe::moe_forward`` /
``uma_qmoe::qwen_moe_forward`` and the Qwen shared-expert block around it.

It is a checker.  Only the test-suite, the smoke entry and the CPU-baseline /
reference arms of the benchmark may import it; the product package never does
and has no CPU fallback.

Pinning: ``tests/golden/make_golden.py`` ran the reference package itself (its
``quantize_q4`` / ``encode_target_tensor`` / ``write_expert_pack`` /
``write_target_pack`` and its ``torch.ops.uma_qmoe.*`` CPU dispatch) on seeded
inputs and stored inputs and outputs in ``tests/golden/*.npz``;
``tests/test_oracle_golden.py`` checks every function below against those
vectors (codecs and routing indices bit-exactly, activations bit-exactly when
the same torch build is used, else within one BF16 ulp).  The reference's own
known-answer vectors (``tests/unit/test_q4.py:19-55``,
``tests/unit/test_target_pack.py:140-166``) are repeated there as well.

Every function cites the reference file:line it follows (paths are relative to
the reference project root).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Sequence

import numpy as np
import torch
import torch.nn.functional as F

GROUP = 128
Q4_MIN, Q4_MAX = -7, 7


# --------------------------------------------------------------------------
# Codecs
# --------------------------------------------------------------------------

def pack_int4(values: np.ndarray) -> np.ndarray:
    """Signed [-7, 7] -> bytes, low nibble first, two's complement.

    Follows ``src/uma_qmoe/q4.py:96-114``.
    """
    flat = np.asarray(values).reshape(-1).astype(np.int16)
    if flat.size == 0:
        raise ValueError("cannot pack an empty Q4 array")
    if flat.min() < Q4_MIN or flat.max() > Q4_MAX:
        raise ValueError("Q4 nibble input is outside [-7, 7]")
    nib = (flat & 0xF).astype(np.uint8)
    if nib.size % 2:
        nib = np.concatenate((nib, np.zeros(1, np.uint8)))
    return (nib[0::2] | (nib[1::2] << 4)).astype(np.uint8)


def unpack_int4(packed: np.ndarray, count: int) -> np.ndarray:
    """Inverse of :func:`pack_int4`; rejects the reserved -8 code and a
    non-zero odd-tail nibble.  Follows ``src/uma_qmoe/q4.py:117-133``."""
    raw = np.frombuffer(bytes(packed), dtype=np.uint8)
    if raw.size != (count + 1) // 2:
        raise ValueError("Q4 packed byte count does not match element count")
    nib = np.empty(raw.size * 2, np.uint8)
    nib[0::2] = raw & 0xF
    nib[1::2] = raw >> 4
    signed = nib.astype(np.int8)
    signed[signed >= 8] -= 16
    out = signed[:count]
    if out.size and out.min() < Q4_MIN:
        raise ValueError("Q4 payload contains the reserved -8 code")
    if count % 2 and int(nib[-1]) != 0:
        raise ValueError("Q4 odd tail padding nibble must be zero")
    return out


def _grouped(flat: np.ndarray, group: int) -> tuple[np.ndarray, int]:
    count = math.ceil(flat.size / group)
    if count * group == flat.size:
        return flat.reshape(count, group), count
    padded = np.zeros(count * group, np.float32)
    padded[: flat.size] = flat
    return padded.reshape(count, group), count


def quantize_q4(values: np.ndarray, group: int = GROUP) -> tuple[np.ndarray, np.ndarray]:
    """Symmetric per-group Q4: scale = max|g| / 7 as float32 (1.0 for an all-zero
    group), codes = clip(rint(g / scale), -7, 7).  Groups run over the
    row-major flattened tensor.  Returns (packed uint8, scales float32).

    Follows ``src/uma_qmoe/q4.py:136-165``.
    """
    flat = np.asarray(values).astype(np.float32, copy=False).reshape(-1)
    if flat.size == 0 or not np.all(np.isfinite(flat)):
        raise ValueError("Q4 source must be non-empty and finite")
    groups, _ = _grouped(flat, group)
    scales = (np.max(np.abs(groups), axis=1) / Q4_MAX).astype("<f4")
    scales[scales == 0] = 1.0
    codes = np.clip(np.rint(groups / scales[:, None]), Q4_MIN, Q4_MAX)
    codes = codes.astype(np.int8).reshape(-1)[: flat.size]
    return pack_int4(codes), scales


def dequantize_q4(packed: np.ndarray, scales: np.ndarray, shape: Sequence[int],
                  group: int = GROUP) -> np.ndarray:
    """codes.astype(float32) * repeat(scales, group).  Follows
    ``src/uma_qmoe/q4.py:168-179``."""
    count = int(np.prod(shape))
    codes = unpack_int4(packed, count).astype(np.float32)
    s = np.frombuffer(bytes(scales), dtype="<f4")
    if not np.all(np.isfinite(s)) or np.any(s <= 0):
        raise ValueError("Q4 scales must be finite and positive")
    return (codes * np.repeat(s, group)[:count]).reshape(shape)


def quantize_q8(values: np.ndarray, group: int = GROUP) -> tuple[np.ndarray, np.ndarray]:
    """Symmetric per-group Q8: scale = max|g| / 127, codes clipped to +-127,
    stored as int8.  Follows ``src/uma_qmoe/target_pack.py:92-112``."""
    flat = np.asarray(values).astype(np.float32, copy=False).reshape(-1)
    if flat.size == 0 or not np.all(np.isfinite(flat)):
        raise ValueError("Q8 source must be non-empty and finite")
    groups, _ = _grouped(flat, group)
    scales = (np.max(np.abs(groups), axis=1) / 127.0).astype("<f4")
    scales[scales == 0] = 1.0
    codes = np.clip(np.rint(groups / scales[:, None]), -127, 127)
    return codes.astype(np.int8).reshape(-1)[: flat.size], scales


def dequantize_q8(codes: np.ndarray, scales: np.ndarray, shape: Sequence[int],
                  group: int = GROUP) -> np.ndarray:
    """Follows ``src/uma_qmoe/target_pack.py:161-175``."""
    count = int(np.prod(shape))
    q = np.frombuffer(bytes(codes), dtype=np.int8).astype(np.float32)
    s = np.frombuffer(bytes(scales), dtype="<f4")
    if q.size != count or s.size != math.ceil(count / group):
        raise ValueError("Q8 payload lengths are invalid")
    return (q * np.repeat(s, group)[:count]).reshape(shape)


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> BF16 bit patterns (uint16).  Follows
    ``src/uma_qmoe/target_pack.py:78-83``."""
    words = np.ascontiguousarray(values, dtype="<f4").view("<u4")
    rounding = np.uint32(0x7FFF) + ((words >> 16) & 1)
    return ((words + rounding) >> 16).astype("<u2")


def bf16_bits_to_f32(bits: np.ndarray, shape: Sequence[int]) -> np.ndarray:
    """Follows ``src/uma_qmoe/target_pack.py:86-89``."""
    words = np.frombuffer(bytes(bits), dtype="<u2").astype("<u4") << 16
    return words.view("<f4").reshape(shape)


# --------------------------------------------------------------------------
# Weight access
# --------------------------------------------------------------------------

@dataclass
class EncodedMatrix:
    """One expert projection in its canonical stored form."""

    encoding: str          # "q4_group128" | "q8_group128" | "bf16_le"
    shape: tuple[int, int]
    data: np.ndarray       # uint8 nibbles / int8 codes / uint16 bf16 bits
    scales: np.ndarray     # float32 (empty for bf16)

    def decode(self) -> np.ndarray:
        """float32 matrix exactly as the reference correctness path sees it
        (``src/uma_qmoe/target_pack.py:144-176``)."""
        if self.encoding == "q4_group128":
            return dequantize_q4(self.data, self.scales, self.shape)
        if self.encoding == "q8_group128":
            return dequantize_q8(self.data, self.scales, self.shape)
        if self.encoding == "bf16_le":
            return bf16_bits_to_f32(self.data, self.shape)
        raise ValueError(self.encoding)


def encode_matrix(values: np.ndarray, encoding: str) -> EncodedMatrix:
    """``encode_target_tensor`` (``src/uma_qmoe/target_pack.py:115-141``)."""
    src = np.asarray(values, dtype=np.float32)
    shape = (int(src.shape[0]), int(src.shape[1]))
    if encoding == "q4_group128":
        data, scales = quantize_q4(src)
    elif encoding == "q8_group128":
        data, scales = quantize_q8(src)
    elif encoding == "bf16_le":
        data, scales = f32_to_bf16_bits(src).reshape(-1), np.zeros(0, np.float32)
    else:
        raise ValueError(encoding)
    return EncodedMatrix(encoding, shape, data, scales)


# expert_number -> (gate, up, down) as EncodedMatrix
ExpertSource = Callable[[int], tuple[EncodedMatrix, EncodedMatrix, EncodedMatrix]]


# --------------------------------------------------------------------------
# Router (third-party arithmetic: Hugging Face transformers, not vendored by the
# reference; call sites src/uma_qmoe/compressed_loader.py:59 and
# src/uma_qmoe/qwen_compressed_loader.py:73; the reference's own restatement is
# benchmarks/runners/capture_qwen_route_trace.py:46-66)
# --------------------------------------------------------------------------

def router_topk(hidden: torch.Tensor, router_weight: torch.Tensor, top_k: int,
                renormalize: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``OlmoeTopKRouter.forward`` / ``Qwen2MoeTopKRouter.forward``:
    logits = linear(x, W) in the activation dtype, softmax in float32 over the
    experts, top-k, optional division by the top-k sum.

    Returns (probabilities [T,E] f32, weights [T,k] f32, indices [T,k] i64).
    """
    x = hidden.reshape(-1, hidden.shape[-1])
    logits = F.linear(x, router_weight)
    probs = F.softmax(logits, dtype=torch.float, dim=-1)
    top, idx = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        top = top / top.sum(dim=-1, keepdim=True)
    return probs, top.to(probs.dtype), idx


# --------------------------------------------------------------------------
# Operator: CPU correctness path
# --------------------------------------------------------------------------

def _expert_mlp_f32(selected: torch.Tensor, gate: np.ndarray, up: np.ndarray,
                    down: np.ndarray) -> torch.Tensor:
    """float32 gate/up linear -> silu(gate) * up -> down linear
    (``src/uma_qmoe/custom_op.py:36-48,325-333``)."""
    gate_up = torch.from_numpy(np.concatenate((gate, up), axis=0))
    g, u = F.linear(selected, gate_up).chunk(2, dim=-1)
    inter = F.silu(g)
    inter.mul_(u)
    return F.linear(inter, torch.from_numpy(np.ascontiguousarray(down)))


def moe_forward(hidden: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                experts: ExpertSource, *, num_experts: int, top_k: int,
                qwen: bool) -> torch.Tensor:
    """The reference's CPU branch of ``_streaming_reference``
    (``src/uma_qmoe/custom_op.py:301-340``) and ``_qwen_streaming_reference``
    (``:465-506``).

    Hit experts are visited in ascending expert number.  For each one the
    selected rows run the MLP in float32; the result is multiplied by the
    routing weight (cast to float32 for OLMoE ``:334``, in its incoming dtype
    for Qwen ``:500``), rounded to the activation dtype and accumulated with
    ``index_add_`` into an accumulator of the activation dtype -- i.e. one
    BF16 rounding of the contribution and one of the running sum per expert.
    """
    flat = hidden.reshape(-1, hidden.shape[-1])
    if indices.shape != weights.shape or tuple(indices.shape) != (flat.shape[0], top_k):
        raise RuntimeError("routes must have shape [tokens, top_k]")
    if indices.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("expert_indices must use int32 or int64")
    if bool((indices < 0).any()) or bool((indices >= num_experts).any()):
        raise RuntimeError("expert_indices contains an invalid expert")
    out = torch.zeros_like(flat)
    mask = F.one_hot(indices.long(), num_classes=num_experts).permute(2, 1, 0)
    hit = torch.greater(mask.sum(dim=(-1, -2)), 0).nonzero()
    for entry in hit:
        e = int(entry[0])
        slots, rows = torch.where(mask[e])
        gate, up, down = (m.decode() for m in experts(e))
        selected = flat.index_select(0, rows).to(torch.float32)
        y = _expert_mlp_f32(selected, gate, up, down)
        if qwen:
            y = y * weights[rows, slots].unsqueeze(-1)
        else:
            y.mul_(weights[rows, slots].to(torch.float32).unsqueeze(-1))
        out.index_add_(0, rows, y.to(out.dtype))
    return out.reshape(hidden.shape)


def qwen_block_forward(hidden: torch.Tensor, router_weight: torch.Tensor,
                       shared_gate_proj: torch.Tensor, shared_up_proj: torch.Tensor,
                       shared_down_proj: torch.Tensor, shared_expert_gate: torch.Tensor,
                       experts: ExpertSource, *, num_experts: int = 60, top_k: int = 4,
                       renormalize: bool = False) -> torch.Tensor:
    """``QuantizedQwenMoEBlock.forward``
    (``src/uma_qmoe/qwen_compressed_loader.py:67-86``): shared expert
    (``Qwen2MoeMLP``: three bias-free ``nn.Linear`` in the activation dtype, so
    each linear output is rounded to BF16), router, routed experts, then
    ``out += sigmoid(linear(x, wg)) * shared``.
    """
    flat = hidden.reshape(-1, hidden.shape[-1])
    shared = F.linear(F.silu(F.linear(flat, shared_gate_proj)) * F.linear(flat, shared_up_proj),
                      shared_down_proj)
    _p, w, idx = router_topk(flat, router_weight, top_k, renormalize)
    routed = moe_forward(flat, idx, w, experts, num_experts=num_experts, top_k=top_k, qwen=True)
    shared = torch.sigmoid(F.linear(flat, shared_expert_gate)) * shared
    routed.add_(shared)
    return routed.reshape(hidden.shape)


def olmoe_block_forward(hidden: torch.Tensor, router_weight: torch.Tensor,
                        experts: ExpertSource, *, num_experts: int = 64, top_k: int = 8,
                        renormalize: bool = False) -> torch.Tensor:
    """``QuantizedMoEBlock.forward`` (``src/uma_qmoe/compressed_loader.py:58-67``)."""
    _p, w, idx = router_topk(hidden, router_weight, top_k, renormalize)
    return moe_forward(hidden, idx, w, experts, num_experts=num_experts, top_k=top_k, qwen=False)


# --------------------------------------------------------------------------
# Routing metadata the native prefill path consumes
# --------------------------------------------------------------------------

def sorted_routes(indices: torch.Tensor, num_experts: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Stable argsort of the flattened expert ids plus ``[E+1]`` offsets
    (``src/uma_qmoe/native_backend.py:531-543``)."""
    flat = indices.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.cat((torch.zeros(1, dtype=torch.int64), torch.cumsum(counts, 0)))
    return order, offsets


# --------------------------------------------------------------------------
# Comparison helper used by every activation parity test
# --------------------------------------------------------------------------

def compare(actual: torch.Tensor, expected: torch.Tensor) -> dict[str, float]:
    a = actual.detach().float().cpu().reshape(-1).double()
    b = expected.detach().float().cpu().reshape(-1).double()
    diff = (a - b).abs()
    denom = float(a.norm() * b.norm())
    cosine = float((a @ b) / denom) if denom > 0 else 1.0
    return {
        "max_abs": float(diff.max()) if diff.numel() else 0.0,
        "p99_abs": float(torch.quantile(diff[:: max(1, diff.numel() // 1_000_000)], 0.99)) if diff.numel() else 0.0,
        "cosine": cosine,
    }
