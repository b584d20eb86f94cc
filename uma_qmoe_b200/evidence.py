"""Kernel evidence in the shape of the reference's control plane.

The reference's validator (``benchmarks/runners/validate_packed_q4_kernel.py:105-336``) runs a fixed workload on an
ExpertPack -- every projection of expert 0 as a linear layer, one decode token and a 32-token prefill over experts
0..7 with weights 0.125 -- and writes a ``packed_q4_kernel_evidence`` document whose gates its contract checker
recomputes from the measurements (``src/uma_qmoe/contracts.py:369-498``).  :func:`measure` runs the same workload on
this package's back end and :func:`build_document` / :func:`check_document` produce and re-check a document with the
same keys, types and gate rules.

Two values cannot be the reference's: its schema (``src/uma_qmoe/schemas/packed_q4_kernel_evidence.schema.json``)
enumerates the platforms ``hip_gfx1151`` / ``cuda_sm121`` and the targets ``halo3`` / ``local-halo`` / ``spark1``; a
B200 document says ``cuda_sm100`` and a target id of the caller's choosing, and names this library's ABI and execution
strategy.  With those four strings added to the schema's enumerations the document validates unchanged.  The
correctness reference is a float32 evaluation of the dequantised experts in torch on the same device (this package
has no CPU path behind the operator).
"""

from __future__ import annotations

import hashlib
import math
import statistics
from datetime import datetime, timezone
from pathlib import Path
from typing import Any

from .formats import ContractError

KIND = "packed_q4_kernel_evidence"
MODEL_ID = "allenai/OLMoE-1B-7B-0125"
ABI = "q4-group128-packed-u8-fp32-scale-bf16-in-bf16-out-sm100-tcgen05-v1"
EXECUTION_STRATEGY = "decode-two-launch-resident-prefill-tcgen05-grouped-gemm-by-index"
ACCEPTANCE = {"max_absolute_error": 1.0, "minimum_cosine_similarity": 0.99}


def nearest_rank(samples: list[float], q: float) -> float:
    ordered = sorted(samples)
    return ordered[max(0, math.ceil(q * len(ordered)) - 1)]


def _passes(result: dict[str, Any]) -> bool:
    return bool(result["finite"] and result["max_absolute_error"] <= ACCEPTANCE["max_absolute_error"]
                and result["cosine_similarity"] >= ACCEPTANCE["minimum_cosine_similarity"])


def build_document(measured: dict[str, Any], *, target_id: str, model_revision: str, expert_pack_sha256: str,
                   platform: str, device_name: str, source_sha256: str, warmup_iterations: int,
                   measured_iterations: int) -> dict[str, Any]:
    """The evidence document for the measurements of :func:`measure` (or any dictionary of the same keys)."""
    samples, prefill_samples = measured["samples_milliseconds"], measured["prefill_samples_milliseconds"]
    cache = measured["cache_summary"]
    gates = {
        "target_architecture": platform == "cuda_sm100",
        "target_compilation": True,
        "direct_packed_input": True,
        "no_dequantized_weight_cache": cache["dequantized_weight_bytes"] == 0,
        "projection_correctness": all(_passes(r) for r in measured["projection_results"]),
        "moe_correctness": _passes(measured["moe_forward"]),
        "prefill_moe_correctness": _passes(measured["prefill_moe_forward"]),
        "performance_mode_executed": len(samples) == measured_iterations,
        "prefill_performance_mode_executed": len(prefill_samples) == measured_iterations,
    }
    gates["overall_passed"] = all(gates.values())
    return {
        "schema_version": 1, "kind": KIND,
        "captured_at": datetime.now(timezone.utc).isoformat(timespec="seconds").replace("+00:00", "Z"),
        "target_id": target_id, "status": "passed" if gates["overall_passed"] else "failed",
        "model": {"model_id": MODEL_ID, "model_revision": model_revision, "expert_pack_sha256": expert_pack_sha256},
        "kernel": {"platform": platform, "device_name": device_name, "source_sha256": source_sha256, "abi": ABI,
                   "execution_strategy": EXECUTION_STRATEGY, "compiled_for_target": True,
                   "reads_packed_weights_directly": True, "full_dequantized_weight_cache": False},
        "workload": {"layer_index": 0, "tokens": 1, "prefill_tokens": measured["prefill_tokens"], "top_k": 8,
                     "unique_experts": 8, "warmup_iterations": warmup_iterations,
                     "measured_iterations": measured_iterations},
        "correctness": {"projection_results": measured["projection_results"], "moe_forward": measured["moe_forward"],
                        "prefill_moe_forward": measured["prefill_moe_forward"], "acceptance": dict(ACCEPTANCE)},
        "performance": {"scope": "single_moe_layer_microbenchmark", "samples_milliseconds": samples,
                        "median_milliseconds": statistics.median(samples), "p95_milliseconds": nearest_rank(samples, 0.95),
                        "prefill_samples_milliseconds": prefill_samples,
                        "prefill_median_milliseconds": statistics.median(prefill_samples),
                        "prefill_p95_milliseconds": nearest_rank(prefill_samples, 0.95),
                        "compressed_cache_tensor_count": cache["tensor_count"],
                        "compressed_cache_bytes": cache["device_storage_bytes"],
                        "dequantized_weight_cache_bytes": cache["dequantized_weight_bytes"], "formal_tps_claim": False},
        "gates": gates,
    }


def check_document(document: dict[str, Any]) -> None:
    """The consistency rules the reference's checker applies to such a document: required keys and constants, each
    projection once, timing summaries recomputed from the samples, every gate recomputed from what was measured,
    overall gate and status derived from the gates.  Raises ``ContractError`` on the first violation."""
    required = {"schema_version", "kind", "captured_at", "target_id", "status", "model", "kernel", "workload",
                "correctness", "performance", "gates"}
    if not isinstance(document, dict) or not required <= set(document):
        raise ContractError("Packed Q4 evidence lacks required fields")
    if document["schema_version"] != 1 or document["kind"] != KIND or document["model"].get("model_id") != MODEL_ID:
        raise ContractError("Packed Q4 evidence has the wrong kind, version or model")
    kernel, workload = document["kernel"], document["workload"]
    correctness, performance, gates = document["correctness"], document["performance"], document["gates"]
    if kernel.get("abi") == ABI and kernel.get("execution_strategy") != EXECUTION_STRATEGY:
        raise ContractError("Packed Q4 fused evidence must declare its execution strategy")
    if workload.get("top_k") != 8 or performance.get("scope") != "single_moe_layer_microbenchmark" \
            or performance.get("formal_tps_claim") is not False or performance.get("dequantized_weight_cache_bytes") != 0:
        raise ContractError("Packed Q4 evidence constants are wrong")
    acceptance = correctness["acceptance"]

    def passes(result: dict[str, Any]) -> bool:
        return bool(result["finite"] and result["max_absolute_error"] <= acceptance["max_absolute_error"]
                    and result["cosine_similarity"] >= acceptance["minimum_cosine_similarity"])
    if sorted(r["name"] for r in correctness["projection_results"]) != ["down_proj", "gate_proj", "up_proj"]:
        raise ContractError("Packed Q4 evidence must cover each projection once")
    for samples_key, median_key, p95_key, what in (
            ("samples_milliseconds", "median_milliseconds", "p95_milliseconds", "timing"),
            ("prefill_samples_milliseconds", "prefill_median_milliseconds", "prefill_p95_milliseconds", "prefill timing")):
        samples = performance.get(samples_key)
        if not isinstance(samples, list) or not samples:
            raise ContractError("Packed Q4 v3 evidence must include a prefill workload")
        if not math.isclose(performance.get(median_key, math.nan), statistics.median(samples), rel_tol=1e-9) or \
                not math.isclose(performance.get(p95_key, math.nan), nearest_rank(samples, 0.95), rel_tol=1e-9):
            raise ContractError(f"Packed Q4 {what} summary does not match samples")
    if workload.get("prefill_tokens", 0) < 2 or not isinstance(correctness.get("prefill_moe_forward"), dict):
        raise ContractError("Packed Q4 v3 evidence must include a prefill workload")
    expected = {
        "target_architecture": kernel["platform"] == "cuda_sm100",
        "target_compilation": kernel["compiled_for_target"],
        "direct_packed_input": kernel["reads_packed_weights_directly"],
        "no_dequantized_weight_cache": not kernel["full_dequantized_weight_cache"]
        and performance["dequantized_weight_cache_bytes"] == 0,
        "projection_correctness": all(passes(r) for r in correctness["projection_results"]),
        "moe_correctness": passes(correctness["moe_forward"]),
        "prefill_moe_correctness": passes(correctness["prefill_moe_forward"]),
        "performance_mode_executed": len(performance["samples_milliseconds"]) == workload["measured_iterations"],
        "prefill_performance_mode_executed": len(performance["prefill_samples_milliseconds"]) == workload["measured_iterations"],
    }
    if any(gates.get(name) != value for name, value in expected.items()):
        raise ContractError("Packed Q4 gate does not match measured evidence")
    overall = all(expected.values())
    if gates.get("overall_passed") != overall:
        raise ContractError("Packed Q4 overall gate is inconsistent")
    if document["status"] != ("passed" if overall else "failed"):
        raise ContractError("Packed Q4 status is inconsistent")


def _agreement(candidate: Any, reference: Any) -> dict[str, Any]:
    import torch
    a, b = candidate.float().flatten(), reference.float().flatten()
    return {"finite": bool(torch.isfinite(a).all()), "max_absolute_error": float((a - b).abs().max()),
            "cosine_similarity": float(torch.nn.functional.cosine_similarity(a, b, dim=0))}


def _tensor_sha256(tensor: Any) -> str:
    import torch
    return hashlib.sha256(tensor.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes()).hexdigest()


def measure(reader: Any, *, device: Any = "cuda:0", warmup_iterations: int = 3, measured_iterations: int = 10) -> dict[str, Any]:
    """Runs the reference validator's workload on a registered pack with this package's back end and returns the
    measurements :func:`build_document` needs.  ``reader``: an open ExpertPack reader of either family."""
    import numpy as np
    import torch

    from . import custom_op, native_backend
    from .formats import PackedTensor, decode
    from .packs import expert_tensor_name
    if warmup_iterations < 1 or measured_iterations < 3:
        raise ContractError("packed Q4 timing requires >=1 warmup and >=3 measured samples")
    backend = native_backend.install_mixed_target_backend()
    handle = custom_op.register_expert_pack(reader)
    device = torch.device(device)

    def dense(name: str) -> Any:
        data, scales, meta = reader.tensor_views(name)
        try:
            packed = PackedTensor("q4_group128", tuple(meta["shape"]), bytes(data), bytes(scales))
        finally:
            data.release()
            scales.release()
        return torch.from_numpy(np.ascontiguousarray(decode(packed))).to(device)

    def time_calls(fn) -> list[float]:
        for _ in range(warmup_iterations):
            fn()
        torch.cuda.synchronize(device)
        samples = []
        for _ in range(measured_iterations):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(); fn(); stop.record()
            stop.synchronize()
            samples.append(float(start.elapsed_time(stop)))
        return samples
    try:
        with torch.inference_mode():
            inputs = {"gate_proj": torch.linspace(-0.5, 0.5, 2048), "up_proj": torch.linspace(0.25, -0.25, 2048),
                      "down_proj": torch.linspace(-0.75, 0.75, 1024)}
            projection_results = []
            for projection, values in inputs.items():
                name = expert_tensor_name(0, 0, projection)
                weight = dense(name).to(torch.bfloat16)
                x = values.reshape(1, -1).to(device=device, dtype=torch.bfloat16)
                result = _agreement(backend.q4_linear(x, handle, name), torch.nn.functional.linear(x, weight))
                result.update({"name": projection, "shape": list(weight.shape)})
                projection_results.append(result)
            experts = [tuple(dense(expert_tensor_name(0, e, p)) for p in ("gate_proj", "up_proj", "down_proj")) for e in range(8)]

            def reference_moe(hidden: Any) -> Any:           # float32, dequantised experts, weights 0.125 each
                x = hidden.float()
                out = torch.zeros_like(x)
                for gate, up, down in experts:
                    out += 0.125 * ((torch.nn.functional.silu(x @ gate.T) * (x @ up.T)) @ down.T)
                return out

            def inputs_for(tokens: int):
                hidden = torch.linspace(-0.5, 0.5, tokens * 2048, device=device).reshape(tokens, 2048).to(torch.bfloat16)
                idx = torch.arange(8, dtype=torch.int64, device=device).reshape(1, 8).repeat(tokens, 1)
                w = torch.full((tokens, 8), 0.125, dtype=torch.bfloat16, device=device)
                return hidden, idx, w
            results, samples = {}, {}
            for key, tokens in (("moe_forward", 1), ("prefill_moe_forward", 32)):
                hidden, idx, w = inputs_for(tokens)
                call = lambda: torch.ops.uma_qmoe.moe_forward(hidden, idx, w, 0, handle, True)
                out = call()
                torch.cuda.synchronize(device)
                results[key] = _agreement(out, reference_moe(hidden))
                results[key]["output_sha256"] = _tensor_sha256(out)
                samples[key] = time_calls(call)
        return {"projection_results": projection_results, "moe_forward": results["moe_forward"],
                "prefill_moe_forward": results["prefill_moe_forward"], "prefill_tokens": 32,
                "samples_milliseconds": samples["moe_forward"], "prefill_samples_milliseconds": samples["prefill_moe_forward"],
                "cache_summary": backend.cache_summary(), "platform": backend.platform,
                "device_name": torch.cuda.get_device_name(device),
                "source_sha256": native_backend.native_kernel_source_sha256()}
    finally:
        custom_op.unregister_expert_pack(handle)


def sha256_file(path: str | Path) -> str:
    digest = hashlib.sha256()
    with open(path, "rb") as stream:
        while chunk := stream.read(8 << 20):
            digest.update(chunk)
    return digest.hexdigest()


__all__ = ["ABI", "EXECUTION_STRATEGY", "build_document", "check_document", "measure", "nearest_rank", "sha256_file"]
