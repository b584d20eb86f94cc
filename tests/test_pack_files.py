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
from uma_qmoe_b200.pack_files import ExpertPackFile, NativeExpertPackFile, NativeTargetPackFile, TargetPackFile
from uma_qmoe_b200.packs import expert_tensor_name

SEED = 20260917
PREFIX = struct.Struct("<8sIIQQ32s32s")
SHAPES = (("gate_proj", (4, 256)), ("up_proj", (4, 256)), ("down_proj", (256, 4)))


class _Readers:
    def __init__(self, expert, target):
        self.Expert, self.Target = expert, target


@pytest.fixture(params=["python", "native"])
def impl(request):
    """Both reader families: the Python ones and the ones on the library's C++ reader (umaq_pack_open); every case
    below must hold for both, with the same messages."""
    return _Readers(ExpertPackFile, TargetPackFile) if request.param == "python" else _Readers(NativeExpertPackFile, NativeTargetPackFile)


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


def test_expert_pack_file_serves_the_writers_bytes(golden_dir, impl):
    with impl.Expert(golden_dir / "tiny.uqmoepk", expected_model_id="allenai/OLMoE-1B-7B-0125") as pack:
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


def test_target_pack_file_serves_all_three_encodings(golden_dir, impl):
    with impl.Target(golden_dir / "tiny.uqmotpk", expected_policy_id="tiny") as pack:
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


def test_expected_identities_are_enforced(golden_dir, impl):
    with pytest.raises(ContractError, match="model id mismatch"):
        impl.Expert(golden_dir / "tiny.uqmoepk", expected_model_id="someone/else")
    with pytest.raises(ContractError, match="model revision mismatch"):
        impl.Target(golden_dir / "tiny.uqmotpk", expected_model_revision="1" * 40)
    with pytest.raises(ContractError, match="policy id mismatch"):
        impl.Target(golden_dir / "tiny.uqmotpk", expected_policy_id="other")


@pytest.mark.parametrize("name", ["tiny.uqmoepk", "tiny.uqmotpk"])
def test_container_level_corruption_is_rejected(golden_dir, tmp_path, name, impl):
    raw = bytearray((golden_dir / name).read_bytes())
    reader = impl.Expert if name.endswith("epk") else impl.Target
    kind = "ExpertPack" if name.endswith("epk") else "TargetPack"

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


def test_rehashed_tampering_of_the_expert_pack_is_rejected(golden_dir, tmp_path, impl):
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

    impl.Expert(edited(lambda h: None)).close()                      # the rebuild itself is faithful
    with pytest.raises(ContractError, match="tensor count is inconsistent"):
        impl.Expert(edited(lambda h: h.__setitem__("tensor_count", 5)))
    with pytest.raises(ContractError, match="not canonical"):
        impl.Expert(edited(lambda h: None, canonical=False))
    with pytest.raises(ContractError, match="quantization contract mismatch"):
        impl.Expert(edited(lambda h: h["quantization"].__setitem__("signed_range", [-8, 7])))
    with pytest.raises(ContractError, match="model identity hash mismatch"):
        impl.Expert(edited(lambda h: h["model"].__setitem__("model_revision", "f" * 40)))
    with pytest.raises(ContractError, match="layout is invalid"):
        impl.Expert(edited(lambda h: h["tensors"][1].__setitem__("packed_offset", h["tensors"][1]["packed_offset"] + 64)))
    with pytest.raises(ContractError, match="effective bpw is invalid"):
        impl.Expert(edited(lambda h: h["tensors"][0].__setitem__("effective_bits_per_weight", 5.0)))
    with pytest.raises(ContractError, match="names must be unique and safe"):
        impl.Expert(edited(lambda h: h["tensors"][1].__setitem__("name", h["tensors"][0]["name"])))

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
        impl.Expert(edited(lambda h: None, reserved_code))
    with pytest.raises(ContractError, match="scales must be finite and positive"):
        impl.Expert(edited(lambda h: None, bad_scale))
    with pytest.raises(ContractError, match="trailing gap must be zero"):
        impl.Expert(edited(lambda h: None, dirty_gap))
    with pytest.raises(ContractError, match="hash mismatch"):
        impl.Expert(edited(lambda h: None, lambda h, p: p.__setitem__(h["tensors"][3]["packed_offset"], 0x11)))


def test_rehashed_tampering_of_the_target_pack_is_rejected(golden_dir, tmp_path, impl):
    magic, header, payload = _split(golden_dir / "tiny.uqmotpk")
    out = tmp_path / "edited.uqmotpk"

    def edited(change):
        h = json.loads(json.dumps(header))
        change(h)
        return _rebuild(out, magic, h, payload)

    impl.Target(edited(lambda h: None)).close()
    with pytest.raises(ContractError, match="encoding tensor counts are inconsistent"):
        impl.Target(edited(lambda h: h["encoding_tensor_counts"].__setitem__("bf16_le", 5)))
    with pytest.raises(ContractError, match="policy identity hash mismatch"):
        impl.Target(edited(lambda h: h["policy"].__setitem__("policy_id", "renamed")))
    with pytest.raises(ContractError, match="every layer exactly once"):
        impl.Target(edited(lambda h: h["policy"]["layer_encodings"].pop("15")))
    with pytest.raises(ContractError, match="unsupported encoding"):
        impl.Target(edited(lambda h: h["policy"]["layer_encodings"].__setitem__("3", "q2_group64")))
    with pytest.raises(ContractError, match="policy identity is invalid"):
        impl.Target(edited(lambda h: h["tensors"][0].__setitem__("encoding", "q8_group128")))
    with pytest.raises(ContractError, match="schema is unsupported"):
        impl.Target(edited(lambda h: h.__setitem__("format", "something_else")))


def test_pack_files_register_with_the_operator_registry(golden_dir, impl):
    from uma_qmoe_b200 import custom_op
    with impl.Target(golden_dir / "tiny.uqmotpk") as pack:
        handle = custom_op.register_target_pack(pack)
        with custom_op.acquire_expert_pack(handle) as reader:
            assert reader is pack and reader.layer_encoding(1) == "q8_group128"
        custom_op.unregister_expert_pack(handle)


def _hand_made_expert_pack(path, tail_nibble: int = 0, scale: float = 0.5):
    """A one-tensor ExpertPack written here byte by byte: shape [1, 3], so the second data byte has a padding
    nibble, and a bits-per-weight value (512 / 3) whose canonical JSON form needs all 17 digits."""
    data = bytes([0x21, 0x03 | (tail_nibble << 4)])
    scales = struct.pack("<f", scale)
    payload = data + bytes(2) + scales + bytes(56)
    triple = {"model_id": "allenai/OLMoE-1B-7B-0125", "model_revision": "0" * 40, "model_manifest_sha256": "0" * 64}
    canonical = lambda doc: json.dumps(doc, sort_keys=True, separators=(",", ":")).encode()
    header = {
        "schema_version": 1,
        "model": dict(triple, model_identity_sha256=hashlib.sha256(canonical(triple)).hexdigest()),
        "quantization": {"bits": 4, "group_size": 128, "nibble_order": "low_first_twos_complement", "rounding": "nearest_even",
                         "scale_dtype": "float32_le", "signed_range": [-7, 7], "zero_point": None},
        "tensor_alignment_bytes": 64, "tensor_count": 1,
        "tensors": [{"name": "model.layers.0.mlp.experts.0.gate_proj.weight", "shape": [1, 3], "element_count": 3,
                     "group_count": 1, "packed_offset": 0, "packed_bytes": 2, "scale_offset": 4, "scale_bytes": 4,
                     "storage_end_offset": 64, "effective_bits_per_weight": 64 * 8 / 3,
                     "tensor_payload_sha256": hashlib.sha256(data + scales).hexdigest()}],
    }
    return _rebuild(path, b"UQMOEPK1", header, payload)


def test_odd_element_count_tail_nibble_and_scales(tmp_path, impl):
    """The remaining rejection cases of the reference's ``tests/unit/test_expert_pack.py:132-168``: a non-zero padding
    nibble behind an odd element count and a NaN scale, each with every hash recomputed."""
    with impl.Expert(_hand_made_expert_pack(tmp_path / "good.uqmoepk")) as pack:
        data, scales, entry = pack.tensor_views("model.layers.0.mlp.experts.0.gate_proj.weight")
        assert bytes(data) == b"\x21\x03" and struct.unpack("<f", bytes(scales)) == (0.5,)
        assert entry["effective_bits_per_weight"] == 512 / 3
        data.release(); scales.release()
    with pytest.raises(ContractError, match="non-zero Q4 tail padding"):
        impl.Expert(_hand_made_expert_pack(tmp_path / "tail.uqmoepk", tail_nibble=1))
    with pytest.raises(ContractError, match="scales must be finite and positive"):
        impl.Expert(_hand_made_expert_pack(tmp_path / "nan.uqmoepk", scale=float("nan")))
    with pytest.raises(ContractError, match="scales must be finite and positive"):
        impl.Expert(_hand_made_expert_pack(tmp_path / "zero.uqmoepk", scale=0.0))


def test_native_sha256_matches_hashlib_on_both_code_paths():
    """The C++ reader's SHA-256, with and without the CPU's SHA extensions, on lengths around the block and padding
    boundaries."""
    import ctypes as C

    from uma_qmoe_b200 import _native
    lib = _native.lib()
    rng = np.random.default_rng(3)
    for n in (0, 1, 55, 56, 57, 63, 64, 65, 119, 120, 128, 4097, 1 << 20):
        data = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        for scalar_only in (0, 1):
            digest = (C.c_ubyte * 32)()
            assert lib.umaq_sha256(data, n, scalar_only, digest) == 0
            assert bytes(digest) == hashlib.sha256(data).digest(), (n, scalar_only)


def test_writers_reproduce_the_reference_writers_files(golden_dir, tmp_path):
    """This package's writers, given the inputs the golden files were made from, must write the same files byte for
    byte as the reference's writers did (prefix, canonical header, payload layout and hashes)."""
    from uma_qmoe_b200.pack_writer import write_expert_pack, write_target_pack
    zeros40, zeros64 = "0" * 40, "0" * 64
    small = [(expert_tensor_name(0, e, p), _source(e, i, s)) for e in range(2) for i, (p, s) in enumerate(SHAPES)]
    info = write_expert_pack(tmp_path / "mine.uqmoepk", small, model_id="allenai/OLMoE-1B-7B-0125", model_revision=zeros40,
                             model_manifest_sha256=zeros64)
    assert (tmp_path / "mine.uqmoepk").read_bytes() == (golden_dir / "tiny.uqmoepk").read_bytes()
    assert info["file_size"] == (golden_dir / "tiny.uqmoepk").stat().st_size
    layered = [(expert_tensor_name(l, e, p), _source(e, i, s)) for l in range(3) for e in range(2)
               for i, (p, s) in enumerate(SHAPES)]
    write_target_pack(tmp_path / "mine.uqmotpk", layered, model_id="allenai/OLMoE-1B-7B-0125", model_revision=zeros40,
                      model_manifest_sha256=zeros64, policy_id="tiny",
                      layer_encodings={i: ("q4_group128", "q8_group128", "bf16_le")[i % 3] for i in range(16)},
                      policy_evidence_sha256=zeros64)
    assert (tmp_path / "mine.uqmotpk").read_bytes() == (golden_dir / "tiny.uqmotpk").read_bytes()
    with pytest.raises(ContractError, match="refusing to overwrite"):
        write_expert_pack(tmp_path / "mine.uqmoepk", small, model_id="x", model_revision=zeros40, model_manifest_sha256=zeros64)
    with pytest.raises(ContractError, match="every layer exactly once"):
        write_target_pack(tmp_path / "other.uqmotpk", layered, model_id="allenai/OLMoE-1B-7B-0125", model_revision=zeros40,
                          model_manifest_sha256=zeros64, policy_id="tiny", layer_encodings={0: "q4_group128"},
                          policy_evidence_sha256=zeros64)
    assert not (tmp_path / "other.uqmotpk").exists() and len(list(tmp_path.iterdir())) == 2    # no temporary files left
