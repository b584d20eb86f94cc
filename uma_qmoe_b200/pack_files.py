"""Readers for the two on-disk containers of quantised experts.

``ExpertPackFile`` reads ``UQMOEPK1`` (all tensors canonical Q4, ``src/uma_qmoe/expert_pack.py:317-556`` in the
reference), ``TargetPackFile`` reads ``UQMOTPK1`` (one encoding per layer out of Q4 / Q8 / BF16,
``src/uma_qmoe/target_pack.py:493-812``).  Both offer what the operator's back end needs from a pack --
``mapping_count == 1``, ``header``, ``tensor_views(name) -> (data, scales, entry)``, ``layer_encoding(i)``,
``close()`` -- so a host can register them with ``register_expert_pack`` / ``register_target_pack`` exactly as it
registers the reference's own readers.

A file is one read-only mapping.  Everything the formats promise is checked when the file is opened, and the
first violation raises ``ContractError``:

* 96-byte prefix ``<8sIIQQ32s32s``: magic, version 1, header length, payload offset (a multiple of 4096, after the
  header), payload length (to the end of the file), SHA-256 of the header bytes and of the payload;
* the header is canonical JSON (``sort_keys``, separators ``,`` and ``:``, no NaN) -- re-serialising the parsed
  document must give the same bytes -- followed by zero padding up to the payload;
* the model identity (and for a TargetPack the policy identity) is the SHA-256 of its canonical JSON triple;
* tensors lie in file order without overlap, data at a multiple of the tensor alignment, scales at the next
  multiple of 4, every gap zero, sizes as the encoding dictates, the recorded bits per weight and the
  per-tensor SHA-256 of data + scales correct;
* Q4 payloads never contain the reserved code -8 and have a zero tail nibble, scales are finite and positive.
"""

from __future__ import annotations

import hashlib
import json
import math
import mmap
import re
import struct
from pathlib import Path
from typing import Any, Mapping, Optional

from .formats import ContractError

_PREFIX = struct.Struct("<8sIIQQ32s32s")
_PAYLOAD_ALIGNMENT = 4096
_SAFE_NAME = re.compile(r"^[A-Za-z0-9_.-]+$")
_EXPERT_NAME = re.compile(r"^model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(down_proj|gate_proj|up_proj)\.weight$")
_HAS_MINUS_EIGHT = bytes(1 if (b & 0x0F) == 8 or (b >> 4) == 8 else 0 for b in range(256))
_QWEN = "Qwen/Qwen1.5-MoE-A2.7B"
ENCODINGS = ("bf16_le", "q4_group128", "q8_group128")


def _canonical(document: Any) -> bytes:
    return json.dumps(document, sort_keys=True, separators=(",", ":"), allow_nan=False).encode("utf-8")


def _identity(document: Mapping[str, Any]) -> str:
    return hashlib.sha256(json.dumps(document, sort_keys=True, separators=(",", ":")).encode("utf-8")).hexdigest()


def _round_up(value: int, multiple: Any, what: str) -> int:
    if isinstance(multiple, bool) or not isinstance(multiple, int) or multiple <= 0:
        raise ContractError(f"{what} alignment must be a positive integer")
    return -(-value // multiple) * multiple


def _positive_int(value: Any) -> bool:
    return isinstance(value, int) and not isinstance(value, bool) and value > 0


class _PackFile:
    """Mapping, prefix, hashes and canonical header shared by both containers."""

    KIND = ""          # "ExpertPack" / "TargetPack", used in messages
    MAGIC = b""
    DATA_KEYS = ("", "")   # names of the entry fields holding the data offset and length

    def __init__(self, path: str | Path, **expected: Optional[str]) -> None:
        self.path = Path(path)
        self._file = None
        self._map: Optional[mmap.mmap] = None
        try:
            self._file = self.path.open("rb")
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        except (OSError, ValueError) as exc:
            self.close()
            raise ContractError(f"cannot map {self.KIND} {self.path}: {exc}") from exc
        self.mapping_count = 1
        try:
            self.header, self.payload_offset, self.payload_length = self._open_checked(expected)
        except BaseException:
            self.close()
            raise
        self._entries = {entry["name"]: entry for entry in self.header["tensors"]}

    # ---- container level --------------------------------------------------------------------------------
    def _open_checked(self, expected: Mapping[str, Optional[str]]) -> tuple[dict[str, Any], int, int]:
        kind, view = self.KIND, self._map
        assert view is not None
        if len(view) < _PREFIX.size:
            raise ContractError(f"{kind} is shorter than its fixed prefix")
        magic, version, header_len, offset, length, header_sha, payload_sha = _PREFIX.unpack_from(view)
        if magic != self.MAGIC or version != 1:
            raise ContractError(f"{kind} magic/version mismatch")
        if offset % _PAYLOAD_ALIGNMENT or offset < _PREFIX.size + header_len:
            raise ContractError(f"{kind} payload offset/alignment is invalid")
        if offset + length != len(view):
            raise ContractError(f"{kind} payload length does not match file size")
        raw = view[_PREFIX.size:_PREFIX.size + header_len]
        if hashlib.sha256(raw).digest() != header_sha:
            raise ContractError(f"{kind} header hash mismatch")
        self._require_zero(_PREFIX.size + header_len, offset, "header padding")
        with memoryview(view)[offset:offset + length] as payload:
            if hashlib.sha256(payload).digest() != payload_sha:
                raise ContractError(f"{kind} payload hash mismatch")
        try:
            header = json.loads(raw)
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise ContractError(f"{kind} header is not canonical JSON") from exc
        try:
            same = _canonical(header) == raw
        except (TypeError, ValueError):
            same = False
        if not same:
            raise ContractError(f"{kind} header JSON is not canonical")
        if not isinstance(header, dict) or header.get("schema_version") != 1:
            raise ContractError(f"{kind} header schema is unsupported")
        model = header.get("model")
        if not isinstance(model, dict):
            raise ContractError(f"{kind} header is incomplete")
        triple = {key: model.get(key, "") for key in ("model_id", "model_revision", "model_manifest_sha256")}
        if model.get("model_identity_sha256") != _identity(triple):
            raise ContractError(f"{kind} model identity hash mismatch")
        for key, label in (("model_id", "model id"), ("model_revision", "model revision"),
                           ("model_manifest_sha256", "model manifest")):
            want = expected.get(f"expected_{key}")
            if want is not None and want != model.get(key):
                raise ContractError(f"{kind} {label} mismatch")
        self._check_document(header, expected)
        self._check_tensors(header, offset, length)
        self._check_totals(header)
        return header, offset, length

    def _require_zero(self, start: int, stop: int, what: str) -> None:
        assert self._map is not None
        if start > stop:
            raise ContractError(f"{self.KIND} {what} has a negative extent")
        if any(self._map[start:stop]):
            raise ContractError(f"{self.KIND} {what} must be zero")

    def _check_document(self, header: dict[str, Any], expected: Mapping[str, Optional[str]]) -> None:
        raise NotImplementedError

    def _entry_rules(self, header: dict[str, Any], entry: dict[str, Any], elements: int) -> tuple[str, int, int]:
        """-> (encoding, data bytes, scale bytes) an entry must have; raises for entry-specific violations."""
        raise NotImplementedError

    def _check_totals(self, header: dict[str, Any]) -> None:
        """Document-level counts that only make sense once every tensor entry has been accepted."""

    # ---- tensor level -----------------------------------------------------------------------------------
    def _check_tensors(self, header: dict[str, Any], payload_offset: int, payload_length: int) -> None:
        kind, view = self.KIND, self._map
        assert view is not None
        entries = header.get("tensors")
        alignment = header.get("tensor_alignment_bytes")
        _round_up(0, alignment, kind)
        if not isinstance(entries, list) or not entries or header.get("tensor_count") != len(entries):
            raise ContractError(f"{kind} tensor count is inconsistent")
        data_key, size_key = self.DATA_KEYS
        seen: set[str] = set()
        end_of_previous = 0
        for entry in entries:
            if not isinstance(entry, dict):
                raise ContractError(f"{kind} tensor header must be an object")
            name = entry.get("name")
            if not isinstance(name, str) or not _SAFE_NAME.fullmatch(name) or name in seen:
                raise ContractError(f"{kind} tensor names must be unique and safe")
            seen.add(name)
            shape = entry.get("shape")
            if not isinstance(shape, list) or not shape or not all(_positive_int(d) for d in shape):
                raise ContractError(f"{kind} tensor {name!r} has invalid shape")
            elements = math.prod(shape)
            encoding, data_bytes, scale_bytes = self._entry_rules(header, entry, elements)
            start, scale_at, end = entry.get(data_key), entry.get("scale_offset"), entry.get("storage_end_offset")
            ok = (entry.get("element_count") == elements and entry.get(size_key) == data_bytes
                  and entry.get("scale_bytes") == scale_bytes and isinstance(start, int) and not isinstance(start, bool)
                  and start % alignment == 0 and start >= end_of_previous
                  and scale_at == _round_up(start + data_bytes, 4, kind)
                  and end == _round_up(scale_at + scale_bytes, alignment, kind) and end <= payload_length)
            if not ok:
                raise ContractError(f"{kind} tensor {name!r} layout is invalid")
            if entry.get("effective_bits_per_weight") != (end - start) * 8 / elements:
                raise ContractError(f"{kind} tensor {name!r} effective bpw is invalid")
            base = payload_offset
            self._require_zero(base + end_of_previous, base + start, f"tensor {name!r} leading gap")
            self._require_zero(base + start + data_bytes, base + scale_at, f"tensor {name!r} data-to-scale gap")
            self._require_zero(base + scale_at + scale_bytes, base + end, f"tensor {name!r} trailing gap")
            with memoryview(view)[base + start:base + start + data_bytes] as data, \
                    memoryview(view)[base + scale_at:base + scale_at + scale_bytes] as scales:
                digest = hashlib.sha256(data)
                digest.update(scales)
                if digest.hexdigest() != entry.get("tensor_payload_sha256"):
                    raise ContractError(f"{kind} tensor {name!r} hash mismatch")
                if encoding == "q4_group128":
                    for at in range(0, len(data), 8 << 20):
                        if bytes(data[at:at + (8 << 20)]).translate(_HAS_MINUS_EIGHT).find(b"\x01") != -1:
                            raise ContractError(f"{kind} tensor {name!r} contains reserved Q4 -8")
                    if elements % 2 and data[-1] >> 4:
                        raise ContractError(f"{kind} tensor {name!r} has non-zero Q4 tail padding")
                for (scale,) in struct.iter_unpack("<f", scales):
                    if not math.isfinite(scale) or scale <= 0:
                        raise ContractError(f"{kind} tensor {name!r} scales must be finite and positive")
            end_of_previous = end
        if end_of_previous != payload_length:
            raise ContractError(f"{kind} payload has unclaimed trailing bytes")

    # ---- what the back end calls --------------------------------------------------------------------------
    def tensor_views(self, name: str) -> tuple[memoryview, memoryview, Mapping[str, Any]]:
        """(data, scales, header entry) of a tensor as views into the mapping; release them before ``close``."""
        entry = self._entries.get(name)
        if entry is None or self._map is None:
            raise ContractError(f"{self.KIND} has no tensor {name!r}")
        data_key, size_key = self.DATA_KEYS
        start = self.payload_offset + entry[data_key]
        scale_at = self.payload_offset + entry["scale_offset"]
        view = memoryview(self._map)
        return view[start:start + entry[size_key]], view[scale_at:scale_at + entry["scale_bytes"]], entry

    def names(self) -> list[str]:
        return list(self._entries)

    def shapes(self) -> dict[str, tuple[int, ...]]:
        return {name: tuple(entry["shape"]) for name, entry in self._entries.items()}

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        if self._file is not None:
            self._file.close()
            self._file = None

    def __enter__(self):
        return self

    def __exit__(self, *_: Any) -> None:
        self.close()


class ExpertPackFile(_PackFile):
    """``UQMOEPK1``: every tensor canonical packed Q4 with float32 scales."""

    KIND, MAGIC, DATA_KEYS = "ExpertPack", b"UQMOEPK1", ("packed_offset", "packed_bytes")

    def __init__(self, path: str | Path, *, expected_model_id: Optional[str] = None,
                 expected_model_revision: Optional[str] = None,
                 expected_model_manifest_sha256: Optional[str] = None) -> None:
        super().__init__(path, expected_model_id=expected_model_id, expected_model_revision=expected_model_revision,
                         expected_model_manifest_sha256=expected_model_manifest_sha256)

    def _check_document(self, header: dict[str, Any], expected: Mapping[str, Optional[str]]) -> None:
        quantization = header.get("quantization")
        if not isinstance(quantization, dict) or not isinstance(header.get("tensors"), list):
            raise ContractError("ExpertPack header is incomplete")
        contract = {"bits": 4, "group_size": quantization.get("group_size"), "nibble_order": "low_first_twos_complement",
                    "rounding": "nearest_even", "scale_dtype": "float32_le", "signed_range": [-7, 7], "zero_point": None}
        if quantization != contract or not _positive_int(quantization.get("group_size")):
            raise ContractError("ExpertPack quantization contract mismatch")

    def _entry_rules(self, header: dict[str, Any], entry: dict[str, Any], elements: int) -> tuple[str, int, int]:
        groups = -(-elements // header["quantization"]["group_size"])
        if entry.get("group_count") != groups:
            raise ContractError(f"ExpertPack tensor {entry.get('name')!r} layout is invalid")
        return "q4_group128", -(-elements // 2), groups * 4

    def layer_encoding(self, layer_index: int) -> str:
        return "q4_group128"


class TargetPackFile(_PackFile):
    """``UQMOTPK1``: one of ``q4_group128`` / ``q8_group128`` / ``bf16_le`` per layer, named by the header's policy."""

    KIND, MAGIC, DATA_KEYS = "TargetPack", b"UQMOTPK1", ("data_offset", "data_bytes")

    def __init__(self, path: str | Path, *, expected_model_id: Optional[str] = None,
                 expected_model_revision: Optional[str] = None,
                 expected_model_manifest_sha256: Optional[str] = None, expected_policy_id: Optional[str] = None) -> None:
        super().__init__(path, expected_model_id=expected_model_id, expected_model_revision=expected_model_revision,
                         expected_model_manifest_sha256=expected_model_manifest_sha256,
                         expected_policy_id=expected_policy_id)

    def _layers(self, header: Mapping[str, Any]) -> tuple[int, int]:
        qwen = header["model"].get("model_id") == _QWEN
        return (24, 60) if qwen else (16, 64)

    def _check_document(self, header: dict[str, Any], expected: Mapping[str, Optional[str]]) -> None:
        if header.get("format") != "mixed_precision_target_pack":
            raise ContractError("TargetPack header schema is unsupported")
        policy = header.get("policy")
        if not isinstance(policy, dict):
            raise ContractError("TargetPack layer policy is invalid")
        want = expected.get("expected_policy_id")
        if want is not None and want != policy.get("policy_id"):
            raise ContractError("TargetPack policy id mismatch")
        layers, _ = self._layers(header)
        table = policy.get("layer_encodings")
        if not isinstance(table, dict) or sorted(table) != sorted(str(i) for i in range(layers)):
            raise ContractError("TargetPack policy must assign every layer exactly once")
        if any(value not in ENCODINGS for value in table.values()):
            raise ContractError("TargetPack policy contains an unsupported encoding")
        policy_id, evidence = policy.get("policy_id"), policy.get("policy_evidence_sha256")
        if not isinstance(policy_id, str) or not policy_id:
            raise ContractError("TargetPack policy id must be non-empty")
        if not isinstance(evidence, str) or not re.fullmatch(r"[0-9a-f]{64}", evidence):
            raise ContractError("TargetPack policy evidence identity must be SHA-256")
        ordered = {str(i): table[str(i)] for i in range(layers)}
        identity = _identity({"policy_id": policy_id, "layer_encodings": ordered, "policy_evidence_sha256": evidence})
        if policy != {"policy_id": policy_id, "layer_encodings": ordered, "policy_evidence_sha256": evidence,
                      "policy_identity_sha256": identity}:
            raise ContractError("TargetPack policy identity hash mismatch")

    def _check_totals(self, header: dict[str, Any]) -> None:
        counts = {encoding: 0 for encoding in ENCODINGS}
        for entry in header["tensors"]:
            counts[entry["encoding"]] += 1
        if header.get("encoding_tensor_counts") != counts:
            raise ContractError("TargetPack encoding tensor counts are inconsistent")

    def _entry_rules(self, header: dict[str, Any], entry: dict[str, Any], elements: int) -> tuple[str, int, int]:
        name = entry.get("name")
        match = _EXPERT_NAME.fullmatch(name) if isinstance(name, str) else None
        if match is None:
            raise ContractError("TargetPack tensor names must be unique fixed OLMoE experts")
        layers, experts = self._layers(header)
        layer, expert, projection = int(match.group(1)), int(match.group(2)), match.group(3)
        encoding = entry.get("encoding")
        if (layer >= layers or expert >= experts or entry.get("layer_index") != layer
                or entry.get("expert_index") != expert or entry.get("projection") != projection
                or encoding != header["policy"]["layer_encodings"][str(layer)]):
            raise ContractError(f"TargetPack tensor {name!r} policy identity is invalid")
        grouped = encoding != "bf16_le"
        groups = -(-elements // 128) if grouped else 0
        if entry.get("group_size") != (128 if grouped else None) or entry.get("group_count") != groups:
            raise ContractError(f"TargetPack tensor {name!r} layout is invalid")
        data_bytes = {"q4_group128": -(-elements // 2), "q8_group128": elements, "bf16_le": elements * 2}[encoding]
        return encoding, data_bytes, groups * 4

    def layer_encoding(self, layer_index: int) -> str:
        layers, _ = self._layers(self.header)
        if not 0 <= layer_index < layers:
            raise ContractError(f"TargetPack layer index must be in [0, {layers - 1}]")
        return self.header["policy"]["layer_encodings"][str(layer_index)]


# ---------------------------------------------------------------------------------------------------------
# The same two readers on the library's native pack reader (umaq_pack_open): one mapping made and checked in
# C++, SHA-256 with the CPU's SHA extensions, tensors served as views into that mapping, and a layer staged
# to the device by a worker thread through pinned chunks while the caller goes on.
# ---------------------------------------------------------------------------------------------------------

class _NativePackFile:
    KIND_ID = 0
    KIND = "ExpertPack"

    def __init__(self, path: str | Path, **expected: Optional[str]) -> None:
        import ctypes as C

        from . import _native
        self.path = Path(path)
        self._lib = _native.lib()
        self._handle = C.c_void_p()
        text = lambda key: None if expected.get(key) is None else str(expected[key]).encode("utf-8")
        code = self._lib.umaq_pack_open(str(self.path).encode("utf-8"), self.KIND_ID, text("expected_model_id"),
                                        text("expected_model_revision"), text("expected_model_manifest_sha256"),
                                        text("expected_policy_id"), C.byref(self._handle))
        if code != 0:
            self._handle = C.c_void_p()
            raise ContractError(self._lib.umaq_last_error().decode("utf-8", "replace"))
        self.mapping_count = 1
        length = C.c_size_t()
        raw = self._lib.umaq_pack_header_json(self._handle, C.byref(length))
        self.header = json.loads(C.string_at(raw, length.value))
        self._names = [entry["name"] for entry in self.header["tensors"]]
        self._entries = {entry["name"]: entry for entry in self.header["tensors"]}

    def _view(self, name: str):
        import ctypes as C

        from . import _native
        if not self._handle:
            raise ContractError(f"{self.KIND} is closed")
        view = _native.PackTensor()
        if self._lib.umaq_pack_tensor_view(self._handle, name.encode("utf-8"), C.byref(view)) != 0:
            raise ContractError(self._lib.umaq_last_error().decode("utf-8", "replace"))
        return view

    def tensor_views(self, name: str) -> tuple[memoryview, memoryview, Mapping[str, Any]]:
        """(data, scales, header entry): read-only views into the native mapping, valid until ``close``."""
        import ctypes as C
        view = self._view(name)
        data = memoryview((C.c_ubyte * view.data_bytes).from_address(view.data)).cast("B").toreadonly()
        scales = (memoryview((C.c_ubyte * view.scale_bytes).from_address(view.scales)).cast("B").toreadonly()
                  if view.scale_bytes else memoryview(b""))
        return data, scales, self._entries[name]

    def names(self) -> list[str]:
        return list(self._names)

    def shapes(self) -> dict[str, tuple[int, ...]]:
        return {name: tuple(entry["shape"]) for name, entry in self._entries.items()}

    def layer_encoding(self, layer_index: int) -> str:
        code = self._lib.umaq_pack_layer_encoding(self._handle, int(layer_index))
        if code < 0:
            raise ContractError(self._lib.umaq_last_error().decode("utf-8", "replace"))
        return ("q4_group128", "q8_group128", "bf16_le")[code]

    def stage_layer_async(self, layer_index: int, destination: Any, device: Any):
        """Start copying layer ``layer_index`` into the device tensors of ``destination`` (a ``DeviceLayer`` of the
        right encoding and shape).  Returns a callable: ``wait(stream) -> host seconds`` blocks until every copy has
        been issued and makes ``stream`` wait for them."""
        import ctypes as C

        import torch
        ticket = C.c_void_p()
        index = torch.device(device).index or 0
        code = self._lib.umaq_stage_layer_async(self._handle, int(layer_index), C.byref(destination.struct()), index,
                                                C.byref(ticket))
        if code != 0:
            raise RuntimeError(self._lib.umaq_last_error().decode("utf-8", "replace"))

        def wait(stream: Any = None) -> float:
            seconds = C.c_double()
            handle = (stream or torch.cuda.current_stream(device)).cuda_stream
            if self._lib.umaq_stage_wait(ticket, C.c_void_p(handle), C.byref(seconds)) != 0:
                raise RuntimeError(self._lib.umaq_last_error().decode("utf-8", "replace"))
            return seconds.value
        return wait

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.umaq_pack_close(self._handle)
            import ctypes as C
            self._handle = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *_: Any) -> None:
        self.close()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass


class NativeExpertPackFile(_NativePackFile):
    """``UQMOEPK1`` through the native reader; same protocol and errors as :class:`ExpertPackFile`."""

    KIND_ID, KIND = 0, "ExpertPack"

    def __init__(self, path: str | Path, *, expected_model_id: Optional[str] = None,
                 expected_model_revision: Optional[str] = None,
                 expected_model_manifest_sha256: Optional[str] = None) -> None:
        super().__init__(path, expected_model_id=expected_model_id, expected_model_revision=expected_model_revision,
                         expected_model_manifest_sha256=expected_model_manifest_sha256)


class NativeTargetPackFile(_NativePackFile):
    """``UQMOTPK1`` through the native reader; same protocol and errors as :class:`TargetPackFile`."""

    KIND_ID, KIND = 1, "TargetPack"

    def __init__(self, path: str | Path, *, expected_model_id: Optional[str] = None,
                 expected_model_revision: Optional[str] = None,
                 expected_model_manifest_sha256: Optional[str] = None, expected_policy_id: Optional[str] = None) -> None:
        super().__init__(path, expected_model_id=expected_model_id, expected_model_revision=expected_model_revision,
                         expected_model_manifest_sha256=expected_model_manifest_sha256,
                         expected_policy_id=expected_policy_id)
