"""Kernel evidence in the reference's control-plane shape (``packed_q4_kernel_evidence``)."""

import copy
import json
from pathlib import Path

import pytest

from uma_qmoe_b200 import evidence
from uma_qmoe_b200.formats import ContractError

ROOT = Path(__file__).resolve().parent.parent
SCHEMA = ROOT / "oracle" / "_ref" / "uma_qmoe" / "schemas" / "packed_q4_kernel_evidence.schema.json"


def _measured():
    ok = {"finite": True, "max_absolute_error": 0.004, "cosine_similarity": 0.99999}
    return {"projection_results": [dict(ok, name=n, shape=s) for n, s in
                                   (("gate_proj", [1024, 2048]), ("up_proj", [1024, 2048]), ("down_proj", [2048, 1024]))],
            "moe_forward": dict(ok, output_sha256="a" * 64), "prefill_moe_forward": dict(ok, output_sha256="b" * 64),
            "prefill_tokens": 32, "samples_milliseconds": [0.031, 0.030, 0.034, 0.029, 0.030],
            "prefill_samples_milliseconds": [0.21, 0.20, 0.22, 0.20, 0.25],
            "cache_summary": {"tensor_count": 192, "device_storage_bytes": 213909504, "dequantized_weight_bytes": 0}}


def _document(**changes):
    measured = _measured()
    measured.update(changes)
    return evidence.build_document(measured, target_id="b200", model_revision="9b0c1aa87e34a20052389dce1f0cf01da783f654",
                                   expert_pack_sha256="c" * 64, platform="cuda_sm100", device_name="NVIDIA B200",
                                   source_sha256="d" * 64, warmup_iterations=3, measured_iterations=5)


def test_document_is_consistent_and_gates_follow_the_measurements():
    doc = _document()
    evidence.check_document(doc)
    assert doc["status"] == "passed" and doc["gates"]["overall_passed"]
    assert doc["performance"]["p95_milliseconds"] == 0.034 and doc["performance"]["median_milliseconds"] == 0.030
    json.dumps(doc, allow_nan=False)
    bad = _document(moe_forward={"finite": True, "max_absolute_error": 3.0, "cosine_similarity": 0.5, "output_sha256": "a" * 64})
    evidence.check_document(bad)                                  # consistent, and failed
    assert bad["status"] == "failed" and not bad["gates"]["moe_correctness"] and not bad["gates"]["overall_passed"]
    short = _document(samples_milliseconds=[0.03, 0.03, 0.03])
    assert not short["gates"]["performance_mode_executed"] and short["status"] == "failed"


@pytest.mark.parametrize("edit,message", [
    (lambda d: d["gates"].__setitem__("moe_correctness", False), "gate does not match"),
    (lambda d: d["performance"].__setitem__("median_milliseconds", 0.02), "timing summary does not match"),
    (lambda d: d["performance"].__setitem__("prefill_p95_milliseconds", 0.2), "prefill timing summary does not match"),
    (lambda d: d.__setitem__("status", "failed"), "status is inconsistent"),
    (lambda d: d["correctness"]["projection_results"].pop(), "each projection once"),
    (lambda d: d["kernel"].__setitem__("execution_strategy", "something-else"), "execution strategy"),
    (lambda d: d["gates"].__setitem__("overall_passed", False), "overall gate is inconsistent"),
    (lambda d: d.pop("workload"), "lacks required fields"),
])
def test_tampered_documents_are_rejected(edit, message):
    doc = copy.deepcopy(_document())
    edit(doc)
    with pytest.raises(ContractError, match=message):
        evidence.check_document(doc)


def test_document_validates_against_the_reference_schema_once_its_enumerations_know_this_platform():
    """The reference's JSON schema, with this platform, target, ABI and strategy added to its four enumerations and
    nothing else changed, accepts the document."""
    jsonschema = pytest.importorskip("jsonschema")
    if not SCHEMA.exists():
        pytest.skip("the reference package is not installed under oracle/_ref")
    schema = json.loads(SCHEMA.read_text())
    doc = _document()
    errors = [e.message for e in jsonschema.Draft202012Validator(schema).iter_errors(doc)]
    assert len(errors) == 4 and all("is not one of" in e for e in errors), errors      # exactly the four enumerations
    schema["properties"]["target_id"]["enum"].append("b200")
    kernel = schema["properties"]["kernel"]["properties"]
    kernel["platform"]["enum"].append("cuda_sm100")
    kernel["abi"]["enum"].append(evidence.ABI)
    kernel["execution_strategy"]["enum"].append(evidence.EXECUTION_STRATEGY)
    jsonschema.Draft202012Validator(schema, format_checker=jsonschema.FormatChecker()).validate(doc)


@pytest.mark.gpu
def test_measured_evidence_on_a_layer_pack_passes_its_gates(tmp_path):
    """The validator's workload on a one-layer OLMoE ExpertPack (written by this package's writer, read by the native
    reader): projections of expert 0 through q4_linear, decode and 32-token prefill through the operator."""
    import torch

    from tests.test_pack_stage_gpu import _write_layer_pack
    from uma_qmoe_b200.pack_files import NativeTargetPackFile
    path, _source = _write_layer_pack(tmp_path, "q4_group128")
    with NativeTargetPackFile(path, expected_policy_id="one-layer") as reader:
        measured = evidence.measure(reader, device="cuda:0", warmup_iterations=2, measured_iterations=5)
    doc = evidence.build_document(measured, target_id="b200", model_revision="0" * 40,
                                  expert_pack_sha256=evidence.sha256_file(path), platform=measured["platform"],
                                  device_name=measured["device_name"], source_sha256=measured["source_sha256"],
                                  warmup_iterations=2, measured_iterations=5)
    evidence.check_document(doc)
    assert doc["status"] == "passed", doc["gates"]
    assert all(r["cosine_similarity"] > 0.9999 for r in doc["correctness"]["projection_results"])
    assert doc["correctness"]["moe_forward"]["max_absolute_error"] <= 2e-2
    assert doc["correctness"]["prefill_moe_forward"]["cosine_similarity"] > 0.9999
    assert doc["performance"]["compressed_cache_tensor_count"] == 192 and torch.cuda.is_available()
