"""Pack-file readers against the two small containers the reference's own writers produced
(``tests/golden/tiny.uqmoepk``, ``tiny.uqmotpk``) and against tampered copies of them; the rejection cases follow
the reference's ``tests/unit/test_expert_pack.py:99-168`` and ``tests/unit/test_target_pack.py:89-110``."""

import hashlib
import json
import struct

import numpy as np
import pytest

from uma_qmoe_b200 import formats, synthetic as syn
from uma_qmoe_b200.formats import ContractError
from uma_qmoe_b200.pack_files import ExpertPackFile, TargetPackFile
from uma_qmoe_b200.packs import expert_tensor_name

SEED = 20260917
PREFIX = struct.Struct("<8sIIQQ32s32s")
SHAPES = (("gate_proj", (4, 256)), ("up_proj", (4, 256)), ("down_proj", (256, 4)))


def _source(expert: int, family: int, shape):
    return syn.normal_bf16((SEED, 9, expert, family), shape, 0.02)


def _split(path):
    raw = path.read_bytes()
    magic, version, header_len, offset, length, _, _ = PREFIX.unpack_from(raw)
    header = json.loads(raw[PREFIX.size:PREFIX.size + header_len])
    return magic, header, bytearray(raw[offset:offset + length])


def _rebuild(path, magic, header, payload, canonical=True):
    """A pack with the given header and payload and every container-level hash recomputed."""
    text = json.dumps(header, sort_keys=True, separators=(",", ":")) if canonical else json.dumps(header, indent=1)
    raw = text.encode()
    offset = -(-(PREFIX.size + len(raw)) // 4096) * 4096
    prefix = PREFIX.pack(magic, 1, len(raw), offset, len(payload), hashlib.sha256(raw).digest(),
                         hashlib.sha256(bytes(payload)).digest())
    path.write_bytes(prefix + raw + bytes(offset - PREFIX.size - len(raw)) + bytes(payload))
    return path


def test_expert_pack_file_serves_the_writers_bytes(golden_dir):
    with ExpertPackFile(golden_dir / "tiny.uqmoepk", expected_model_id="allenai/OLMoE-1B-7B-0125") as pack:
        assert pack.mapping_count == 1 and pack.layer_encoding(7) == "q4_group128"
        assert pack.header["quantization"]["group_size"] == 128
        assert len(pack.names()) == 6
        for expert in range(2):
            for family, (projection, shape) in enumerate(SHAPES):
                data, scales, entry = pack.tensor_views(expert_tensor_name(0, expert, projection))
                want = formats.encode(_source(expert, family, shape), "q4_group128")
                assert bytes(data) == bytes(want.data) and bytes(scales) == bytes(want.scales)
                assert tuple(entry["shape"]) == shape
                data.release(); scales.release()
        with pytest.raises(ContractError, match="has no tensor"):
            pack.tensor_views("model.layers.0.mlp.experts.9.gate_proj.weight")


def test_target_pack_file_serves_all_three_encodings(golden_dir):
    with TargetPackFile(golden_dir / "tiny.uqmotpk", expected_policy_id="tiny") as pack:
        assert pack.mapping_count == 1
        assert [pack.layer_encoding(i) for i in range(3)] == ["q4_group128", "q8_group128", "bf16_le"]
        with pytest.raises(ContractError, match="layer index"):
            pack.layer_encoding(16)
        assert pack.header["encoding_tensor_counts"] == {"bf16_le": 6, "q4_group128": 6, "q8_group128": 6}
        for layer in range(3):
            encoding = pack.layer_encoding(layer)
            for expert in range(2):
                for family, (projection, shape) in enumerate(SHAPES):
                    data, scales, entry = pack.tensor_views(expert_tensor_name(layer, expert, projection))
                    want = formats.encode(_source(expert, family, shape), encoding)
                    assert bytes(data) == bytes(want.data), (layer, expert, projection)
                    assert bytes(scales) == bytes(want.scales or b"")
                    assert entry["encoding"] == encoding
                    data.release(); scales.release()


def test_expected_identities_are_enforced(golden_dir):
    with pytest.raises(ContractError, match="model id mismatch"):
        ExpertPackFile(golden_dir / "tiny.uqmoepk", expected_model_id="someone/else")
    with pytest.raises(ContractError, match="model revision mismatch"):
        TargetPackFile(golden_dir / "tiny.uqmotpk", expected_model_revision="1" * 40)
    with pytest.raises(ContractError, match="policy id mismatch"):
        TargetPackFile(golden_dir / "tiny.uqmotpk", expected_policy_id="other")


@pytest.mark.parametrize("name,reader", [("tiny.uqmoepk", ExpertPackFile), ("tiny.uqmotpk", TargetPackFile)])
def test_container_level_corruption_is_rejected(golden_dir, tmp_path, name, reader):
    raw = bytearray((golden_dir / name).read_bytes())
    kind = "ExpertPack" if reader is ExpertPackFile else "TargetPack"

    def damaged(edit):
        copy = bytearray(raw)
        edit(copy)
        path = tmp_path / "damaged.bin"
        path.write_bytes(bytes(copy))
        return path

    with pytest.raises(ContractError, match="payload hash mismatch"):
        reader(damaged(lambda b: b.__setitem__(len(b) - 70, b[len(b) - 70] ^ 1)))
    with pytest.raises(ContractError, match="header hash mismatch"):
        reader(damaged(lambda b: b.__setitem__(PREFIX.size + 5, b[PREFIX.size + 5] ^ 1)))
    with pytest.raises(ContractError, match="magic/version mismatch"):
        reader(damaged(lambda b: b.__setitem__(0, ord("X"))))
    with pytest.raises(ContractError, match="payload length does not match file size"):
        reader(damaged(lambda b: b.extend(b"\0")))
    _, _, header_len, offset, _, _, _ = PREFIX.unpack_from(raw)
    assert PREFIX.size + header_len < offset                              # there is padding to dirty
    with pytest.raises(ContractError, match="header padding must be zero"):
        reader(damaged(lambda b: b.__setitem__(offset - 1, 1)))
    short = tmp_path / "short.bin"
    short.write_bytes(bytes(raw[:40]))
    with pytest.raises(ContractError, match=f"{kind} is shorter than its fixed prefix"):
        reader(short)
    with pytest.raises(ContractError, match="cannot map"):
        reader(tmp_path / "missing.bin")


def test_rehashed_tampering_of_the_expert_pack_is_rejected(golden_dir, tmp_path):
    """The container hashes alone are not trusted: documents and payloads that were edited and re-hashed."""
    magic, header, payload = _split(golden_dir / "tiny.uqmoepk")
    out = tmp_path / "edited.uqmoepk"

    def edited(change, payload_change=None, canonical=True):
        h = json.loads(json.dumps(header))
        p = bytearray(payload)
        change(h)
        if payload_change:
            payload_change(h, p)
        return _rebuild(out, magic, h, p, canonical)

    ExpertPackFile(edited(lambda h: None)).close()                      # the rebuild itself is faithful
    with pytest.raises(ContractError, match="tensor count is inconsistent"):
        ExpertPackFile(edited(lambda h: h.__setitem__("tensor_count", 5)))
    with pytest.raises(ContractError, match="not canonical"):
        ExpertPackFile(edited(lambda h: None, canonical=False))
    with pytest.raises(ContractError, match="quantization contract mismatch"):
        ExpertPackFile(edited(lambda h: h["quantization"].__setitem__("signed_range", [-8, 7])))
    with pytest.raises(ContractError, match="model identity hash mismatch"):
        ExpertPackFile(edited(lambda h: h["model"].__setitem__("model_revision", "f" * 40)))
    with pytest.raises(ContractError, match="layout is invalid"):
        ExpertPackFile(edited(lambda h: h["tensors"][1].__setitem__("packed_offset", h["tensors"][1]["packed_offset"] + 64)))
    with pytest.raises(ContractError, match="effective bpw is invalid"):
        ExpertPackFile(edited(lambda h: h["tensors"][0].__setitem__("effective_bits_per_weight", 5.0)))
    with pytest.raises(ContractError, match="names must be unique and safe"):
        ExpertPackFile(edited(lambda h: h["tensors"][1].__setitem__("name", h["tensors"][0]["name"])))

    def tensor_hash(h, p, index):
        e = h["tensors"][index]
        body = bytes(p[e["packed_offset"]:e["packed_offset"] + e["packed_bytes"]])
        scales = bytes(p[e["scale_offset"]:e["scale_offset"] + e["scale_bytes"]])
        e["tensor_payload_sha256"] = hashlib.sha256(body + scales).hexdigest()

    def reserved_code(h, p):            # a -8 nibble with every hash recomputed
        p[h["tensors"][0]["packed_offset"]] = 0x08
        tensor_hash(h, p, 0)

    def bad_scale(h, p):
        at = h["tensors"][2]["scale_offset"]
        p[at:at + 4] = struct.pack("<f", -1.0)
        tensor_hash(h, p, 2)

    def dirty_gap(h, p):
        e = h["tensors"][0]
        p[e["scale_offset"] + e["scale_bytes"]] = 7

    with pytest.raises(ContractError, match="contains reserved Q4 -8"):
        ExpertPackFile(edited(lambda h: None, reserved_code))
    with pytest.raises(ContractError, match="scales must be finite and positive"):
        ExpertPackFile(edited(lambda h: None, bad_scale))
    with pytest.raises(ContractError, match="trailing gap must be zero"):
        ExpertPackFile(edited(lambda h: None, dirty_gap))
    with pytest.raises(ContractError, match="hash mismatch"):
        ExpertPackFile(edited(lambda h: None, lambda h, p: p.__setitem__(h["tensors"][3]["packed_offset"], 0x11)))


def test_rehashed_tampering_of_the_target_pack_is_rejected(golden_dir, tmp_path):
    magic, header, payload = _split(golden_dir / "tiny.uqmotpk")
    out = tmp_path / "edited.uqmotpk"

    def edited(change):
        h = json.loads(json.dumps(header))
        change(h)
        return _rebuild(out, magic, h, payload)

    TargetPackFile(edited(lambda h: None)).close()
    with pytest.raises(ContractError, match="encoding tensor counts are inconsistent"):
        TargetPackFile(edited(lambda h: h["encoding_tensor_counts"].__setitem__("bf16_le", 5)))
    with pytest.raises(ContractError, match="policy identity hash mismatch"):
        TargetPackFile(edited(lambda h: h["policy"].__setitem__("policy_id", "renamed")))
    with pytest.raises(ContractError, match="every layer exactly once"):
        TargetPackFile(edited(lambda h: h["policy"]["layer_encodings"].pop("15")))
    with pytest.raises(ContractError, match="unsupported encoding"):
        TargetPackFile(edited(lambda h: h["policy"]["layer_encodings"].__setitem__("3", "q2_group64")))
    with pytest.raises(ContractError, match="policy identity is invalid"):
        TargetPackFile(edited(lambda h: h["tensors"][0].__setitem__("encoding", "q8_group128")))
    with pytest.raises(ContractError, match="schema is unsupported"):
        TargetPackFile(edited(lambda h: h.__setitem__("format", "something_else")))


def test_pack_files_register_with_the_operator_registry(golden_dir):
    from uma_qmoe_b200 import custom_op
    with TargetPackFile(golden_dir / "tiny.uqmotpk") as pack:
        handle = custom_op.register_target_pack(pack)
        with custom_op.acquire_expert_pack(handle) as reader:
            assert reader is pack and reader.layer_encoding(1) == "q8_group128"
        custom_op.unregister_expert_pack(handle)
