"""Writers of the two pack containers, byte-compatible with the reference's
``write_expert_pack`` (``src/uma_qmoe/expert_pack.py:169-314``) and ``write_target_pack``
(``src/uma_qmoe/target_pack.py:300-484``): the same prefix, canonical header and payload layout, so that
either project's readers open either project's files.

The tensors arrive as an iterable of ``(name, values)`` where ``values`` is a float array (encoded here with the
host codecs of :mod:`formats`) or an already encoded :class:`formats.PackedTensor` (for instance bytes the device
packer produced).  The payload is streamed to a temporary file next to the destination while its hash is taken,
then prefix, header and payload are joined; an existing destination is never overwritten.
"""

from __future__ import annotations

import hashlib
import json
import os
import re
import struct
import tempfile
from pathlib import Path
from typing import Any, Iterable, Mapping, Optional

from .formats import ENCODINGS, GROUP_SIZE, ContractError, PackedTensor, encode

_PREFIX = struct.Struct("<8sIIQQ32s32s")
_PAYLOAD_ALIGNMENT = 4096
_TENSOR_ALIGNMENT = 64
_NAME = re.compile(r"^model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(down_proj|gate_proj|up_proj)\.weight$")
_QWEN = "Qwen/Qwen1.5-MoE-A2.7B"
_Q4_CONTRACT = {"bits": 4, "group_size": GROUP_SIZE, "nibble_order": "low_first_twos_complement", "rounding": "nearest_even",
                "scale_dtype": "float32_le", "signed_range": [-7, 7], "zero_point": None}
_ENCODING_CONTRACTS = {
    "bf16_le": {"bits": 16, "byte_order": "little"},
    "q4_group128": _Q4_CONTRACT,
    "q8_group128": {"bits": 8, "group_size": GROUP_SIZE, "rounding": "nearest_even", "scale_dtype": "float32_le",
                    "signed_range": [-127, 127], "zero_point": None},
}


def _canonical(document: Any) -> bytes:
    return json.dumps(document, sort_keys=True, separators=(",", ":"), allow_nan=False).encode("utf-8")


def _sha(document: Any) -> str:
    return hashlib.sha256(_canonical(document)).hexdigest()


def _up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


def _model_block(model_id: str, model_revision: str, model_manifest_sha256: str, kind: str) -> dict[str, str]:
    if not re.fullmatch(r"[0-9a-f]{40}", model_revision):
        raise ContractError(f"{kind} model revision must be a lowercase git SHA")
    if not re.fullmatch(r"[0-9a-f]{64}", model_manifest_sha256):
        raise ContractError(f"{kind} model manifest identity must be SHA-256")
    triple = {"model_id": model_id, "model_revision": model_revision, "model_manifest_sha256": model_manifest_sha256}
    return dict(triple, model_identity_sha256=_sha(triple))


class _Payload:
    """The payload as it grows: a temporary file, its running hash and its length."""

    def __init__(self, target: Path, alignment: int) -> None:
        if isinstance(alignment, bool) or not isinstance(alignment, int) or alignment <= 0:
            raise ContractError("pack alignment must be a positive integer")
        self.alignment = alignment
        self.stream = tempfile.NamedTemporaryFile(prefix=f".{target.name}.", suffix=".payload", dir=target.parent, delete=False)
        self.path = Path(self.stream.name)
        self.digest = hashlib.sha256()
        self.size = 0

    def write(self, data: bytes) -> None:
        self.stream.write(data)
        self.digest.update(data)
        self.size += len(data)

    def pad_to(self, multiple: int) -> int:
        self.write(bytes(_up(self.size, multiple) - self.size))
        return self.size

    def add(self, tensor: PackedTensor) -> dict[str, int]:
        """Append one tensor: data at a multiple of the tensor alignment, scales at the next multiple of 4, zero
        padding to the next tensor boundary.  Returns the offsets the header records."""
        start = self.pad_to(self.alignment)
        self.write(tensor.data)
        scale_at = self.pad_to(4)
        self.write(tensor.scales)
        end = self.pad_to(self.alignment)
        return {"start": start, "scale_offset": scale_at, "storage_end_offset": end}


def _finish(target: Path, magic: bytes, header: dict[str, Any], payload: _Payload) -> dict[str, Any]:
    raw = _canonical(header)
    offset = _up(_PREFIX.size + len(raw), _PAYLOAD_ALIGNMENT)
    prefix = _PREFIX.pack(magic, 1, len(raw), offset, payload.size, hashlib.sha256(raw).digest(), payload.digest.digest())
    payload.stream.close()
    joined = target.with_name(f".{target.name}.joining")
    try:
        with joined.open("xb") as out, payload.path.open("rb") as body:
            out.write(prefix)
            out.write(raw)
            out.write(bytes(offset - _PREFIX.size - len(raw)))
            while chunk := body.read(8 << 20):
                out.write(chunk)
            out.flush()
            os.fsync(out.fileno())
        os.link(joined, target)                    # fails if the destination appeared meanwhile
    finally:
        joined.unlink(missing_ok=True)
        payload.path.unlink(missing_ok=True)
    return {"path": str(target), "header": header, "payload_offset": offset, "payload_length": payload.size,
            "header_sha256": hashlib.sha256(raw).hexdigest(), "payload_sha256": payload.digest.hexdigest(),
            "file_size": offset + payload.size}


def _encoded(values: Any, encoding: str, name: str) -> PackedTensor:
    if isinstance(values, PackedTensor):
        if values.encoding != encoding:
            raise ContractError(f"tensor {name!r} is encoded as {values.encoding}, the layer needs {encoding}")
        return values
    if hasattr(values, "detach"):
        values = values.detach().float().cpu().numpy()
    return encode(values, encoding)


def write_expert_pack(destination: str | Path, tensors: Iterable[tuple[str, Any]], *, model_id: str, model_revision: str,
                      model_manifest_sha256: str, tensor_alignment_bytes: int = _TENSOR_ALIGNMENT) -> dict[str, Any]:
    """One immutable ``UQMOEPK1`` file: every tensor canonical packed Q4 with float32 group-128 scales."""
    target = Path(destination)
    model = _model_block(model_id, model_revision, model_manifest_sha256, "ExpertPack")
    target.parent.mkdir(parents=True, exist_ok=True)
    if target.exists():
        raise ContractError(f"refusing to overwrite existing ExpertPack {target}")
    payload = _Payload(target, tensor_alignment_bytes)
    entries, seen = [], set()
    try:
        for name, values in tensors:
            if not isinstance(name, str) or not re.fullmatch(r"[A-Za-z0-9_.-]+", name) or name in seen:
                raise ContractError(f"invalid or duplicate ExpertPack tensor name {name!r}")
            seen.add(name)
            tensor = _encoded(values, "q4_group128", name)
            at = payload.add(tensor)
            count = tensor.element_count
            entries.append({"name": name, "shape": list(tensor.shape), "element_count": count,
                            "group_count": -(-count // GROUP_SIZE), "packed_offset": at["start"],
                            "packed_bytes": len(tensor.data), "scale_offset": at["scale_offset"],
                            "scale_bytes": len(tensor.scales), "storage_end_offset": at["storage_end_offset"],
                            "effective_bits_per_weight": (at["storage_end_offset"] - at["start"]) * 8 / count,
                            "tensor_payload_sha256": hashlib.sha256(tensor.data + tensor.scales).hexdigest()})
        if not entries:
            raise ContractError("ExpertPack must contain at least one tensor")
        header = {"schema_version": 1, "format": "canonical_q4_symmetric_grouped", "model": model,
                  "quantization": dict(_Q4_CONTRACT), "tensor_alignment_bytes": tensor_alignment_bytes,
                  "tensor_count": len(entries), "tensors": entries}
        return _finish(target, b"UQMOEPK1", header, payload)
    except BaseException:
        payload.stream.close()
        payload.path.unlink(missing_ok=True)
        raise


def write_target_pack(destination: str | Path, tensors: Iterable[tuple[str, Any]], *, model_id: str, model_revision: str,
                      model_manifest_sha256: str, policy_id: str, layer_encodings: Mapping[int, str],
                      policy_evidence_sha256: str, tensor_alignment_bytes: int = _TENSOR_ALIGNMENT) -> dict[str, Any]:
    """One immutable ``UQMOTPK1`` file: each layer's experts in the encoding the policy assigns to the layer."""
    target = Path(destination)
    model = _model_block(model_id, model_revision, model_manifest_sha256, "TargetPack")
    layers, experts = (24, 60) if model_id == _QWEN else (16, 64)
    if not isinstance(policy_id, str) or not policy_id:
        raise ContractError("TargetPack policy id must be non-empty")
    if sorted(layer_encodings) != list(range(layers)):
        raise ContractError("TargetPack policy must assign every layer exactly once")
    if any(value not in ENCODINGS for value in layer_encodings.values()):
        raise ContractError("TargetPack policy contains an unsupported encoding")
    if not re.fullmatch(r"[0-9a-f]{64}", policy_evidence_sha256):
        raise ContractError("TargetPack policy evidence identity must be SHA-256")
    table = {str(i): layer_encodings[i] for i in range(layers)}
    policy = {"policy_id": policy_id, "layer_encodings": table, "policy_evidence_sha256": policy_evidence_sha256}
    policy["policy_identity_sha256"] = _sha(policy)
    target.parent.mkdir(parents=True, exist_ok=True)
    if target.exists():
        raise ContractError(f"refusing to overwrite existing TargetPack {target}")
    payload = _Payload(target, tensor_alignment_bytes)
    entries, seen = [], set()
    try:
        for name, values in tensors:
            match = _NAME.fullmatch(name) if isinstance(name, str) else None
            if match is None or name in seen:
                raise ContractError(f"unexpected or duplicate TargetPack tensor name {name!r}")
            seen.add(name)
            layer, expert = int(match.group(1)), int(match.group(2))
            if layer >= layers or expert >= experts:
                raise ContractError(f"TargetPack tensor identity is out of range: {name!r}")
            encoding = layer_encodings[layer]
            tensor = _encoded(values, encoding, name)
            at = payload.add(tensor)
            count = tensor.element_count
            grouped = encoding != "bf16_le"
            entries.append({"name": name, "layer_index": layer, "expert_index": expert, "projection": match.group(3),
                            "encoding": encoding, "shape": list(tensor.shape), "element_count": count,
                            "group_size": GROUP_SIZE if grouped else None,
                            "group_count": -(-count // GROUP_SIZE) if grouped else 0, "data_offset": at["start"],
                            "data_bytes": len(tensor.data), "scale_offset": at["scale_offset"],
                            "scale_bytes": len(tensor.scales), "storage_end_offset": at["storage_end_offset"],
                            "effective_bits_per_weight": (at["storage_end_offset"] - at["start"]) * 8 / count,
                            "tensor_payload_sha256": hashlib.sha256(tensor.data + tensor.scales).hexdigest()})
        if not entries:
            raise ContractError("TargetPack must contain at least one tensor")
        header = {"schema_version": 1, "format": "mixed_precision_target_pack", "model": model,
                  "encodings": {key: dict(value) for key, value in _ENCODING_CONTRACTS.items()}, "policy": policy,
                  "encoding_tensor_counts": {e: sum(item["encoding"] == e for item in entries) for e in sorted(ENCODINGS)},
                  "tensor_alignment_bytes": tensor_alignment_bytes, "tensor_count": len(entries), "tensors": entries}
        return _finish(target, b"UQMOTPK1", header, payload)
    except BaseException:
        payload.stream.close()
        payload.path.unlink(missing_ok=True)
        raise


__all__ = ["write_expert_pack", "write_target_pack"]
