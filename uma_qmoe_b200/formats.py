"""Host-side codecs for the three canonical expert-weight encodings.

Byte layouts (the contract shared with the reference's ExpertPack / TargetPack):

* ``q4_group128`` -- symmetric 4-bit codes in [-7, 7] (-8 is reserved), two per
  byte, element 2i in the low nibble, two's complement; one little-endian
  float32 scale per 128 consecutive elements of the row-major tensor
  (``src/uma_qmoe/q4.py:96-165`` in the reference).
* ``q8_group128`` -- int8 codes in [-127, 127], same scale grouping
  (``src/uma_qmoe/target_pack.py:92-112``).
* ``bf16_le`` -- little-endian BF16 words, no scales (``target_pack.py:78-89``).

The device-side packer (``umaq_quantize_groups`` in the native library) writes
the same bytes; these numpy versions serve small tensors and the CPU tests.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

GROUP_SIZE = 128
ENCODINGS = ("q4_group128", "q8_group128", "bf16_le")
ENC_Q4, ENC_Q8, ENC_BF16 = 0, 1, 2          # native enum values
ENCODING_ID = {"q4_group128": ENC_Q4, "q8_group128": ENC_Q8, "bf16_le": ENC_BF16}


class ContractError(ValueError):
    """Same role as the reference's ``contracts.ContractError`` (a ``ValueError``)."""


@dataclass(frozen=True)
class PackedTensor:
    encoding: str
    shape: tuple[int, ...]
    data: bytes
    scales: bytes = b""

    @property
    def element_count(self) -> int:
        return int(np.prod(self.shape))


def row_bytes(encoding: str, k: int) -> int:
    return {"q4_group128": k // 2, "q8_group128": k, "bf16_le": 2 * k}[encoding]


def _group_view(flat: np.ndarray) -> np.ndarray:
    n = -(-flat.size // GROUP_SIZE)
    if n * GROUP_SIZE != flat.size:
        grown = np.zeros(n * GROUP_SIZE, np.float32)
        grown[: flat.size] = flat
        flat = grown
    return flat.reshape(n, GROUP_SIZE)


def _symmetric_codes(values: np.ndarray, qmax: int) -> tuple[np.ndarray, np.ndarray]:
    flat = np.asarray(values, dtype=np.float32).reshape(-1)
    if flat.size == 0:
        raise ContractError("cannot quantize an empty tensor")
    if not np.isfinite(flat).all():
        raise ContractError("quantizer input must be finite")
    g = _group_view(flat)
    scale = (np.abs(g).max(axis=1) / qmax).astype("<f4")
    scale[scale == 0] = 1.0
    q = np.rint(g / scale[:, None])
    np.clip(q, -qmax, qmax, out=q)
    return q.astype(np.int8).reshape(-1)[: flat.size], scale


def nibbles_to_bytes(codes: np.ndarray) -> bytes:
    c = np.asarray(codes).reshape(-1)
    if c.size == 0:
        raise ContractError("cannot pack an empty Q4 array")
    if not np.issubdtype(c.dtype, np.integer):
        raise ContractError("Q4 nibble input must be integer")
    if c.min() < -7 or c.max() > 7:
        raise ContractError("Q4 nibble input is outside [-7, 7]")
    u = (c.astype(np.int16) & 0xF).astype(np.uint8)
    if u.size & 1:
        u = np.append(u, np.uint8(0))
    return (u[0::2] | (u[1::2] << 4)).tobytes()


def bytes_to_nibbles(payload: bytes | memoryview, count: int) -> np.ndarray:
    raw = np.frombuffer(payload, dtype=np.uint8)
    if raw.size != (count + 1) // 2:
        raise ContractError("Q4 packed byte count does not match element count")
    both = np.empty(raw.size * 2, np.int8)
    both[0::2] = (raw & 0xF).astype(np.int8)
    both[1::2] = (raw >> 4).astype(np.int8)
    both[both > 7] -= 16
    if (both[:count] == -8).any():
        raise ContractError("Q4 payload contains the reserved -8 code")
    if count & 1 and both[-1] != 0:
        raise ContractError("Q4 odd tail padding nibble must be zero")
    return both[:count]


def encode(values: np.ndarray, encoding: str) -> PackedTensor:
    src = np.asarray(values)
    shape = tuple(int(d) for d in src.shape)
    if encoding == "q4_group128":
        codes, scale = _symmetric_codes(src, 7)
        return PackedTensor(encoding, shape, nibbles_to_bytes(codes), scale.tobytes())
    if encoding == "q8_group128":
        codes, scale = _symmetric_codes(src, 127)
        return PackedTensor(encoding, shape, codes.tobytes(), scale.tobytes())
    if encoding == "bf16_le":
        f = np.ascontiguousarray(src, dtype="<f4")
        if f.size == 0 or not np.isfinite(f).all():
            raise ContractError("BF16 source must be non-empty and finite")
        w = f.view("<u4")
        bits = ((w + (np.uint32(0x7FFF) + ((w >> 16) & 1))) >> 16).astype("<u2")
        return PackedTensor(encoding, shape, bits.tobytes())
    raise ContractError(f"unsupported encoding {encoding!r}")


def _checked_scales(payload: bytes, groups: int) -> np.ndarray:
    s = np.frombuffer(payload, dtype="<f4")
    if s.size != groups:
        raise ContractError("scale count does not match the group count")
    if not np.isfinite(s).all() or (s <= 0).any():
        raise ContractError("scales must be finite and positive")
    return s


def decode(t: PackedTensor) -> np.ndarray:
    """float32 tensor a packed tensor stands for."""
    n = t.element_count
    groups = -(-n // GROUP_SIZE)
    if t.encoding == "q4_group128":
        q = bytes_to_nibbles(t.data, n).astype(np.float32)
        s = _checked_scales(t.scales, groups)
        return (q * np.repeat(s, GROUP_SIZE)[:n]).reshape(t.shape)
    if t.encoding == "q8_group128":
        if len(t.data) != n:
            raise ContractError("Q8 payload length is invalid")
        q = np.frombuffer(t.data, dtype=np.int8).astype(np.float32)
        s = _checked_scales(t.scales, groups)
        return (q * np.repeat(s, GROUP_SIZE)[:n]).reshape(t.shape)
    if t.encoding == "bf16_le":
        if len(t.data) != 2 * n or t.scales:
            raise ContractError("BF16 payload layout is invalid")
        return (np.frombuffer(t.data, dtype="<u2").astype("<u4") << 16).view("<f4").reshape(t.shape)
    raise ContractError(f"unsupported encoding {t.encoding!r}")
