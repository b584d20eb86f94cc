"""Fixed-model hosts built from a checkpoint directory and one pack file.

Counterparts of the reference's ``load_fixed_olmoe`` (``src/uma_qmoe/compressed_loader.py:179-330``) and
``load_fixed_qwen`` (``src/uma_qmoe/qwen_compressed_loader.py:143-303``), same arguments, same order of checks and
the same evidence keys, for the ``cuda_sm100`` platform:

1. the directory's ``config.json`` must describe the fixed architecture (model type, layers, experts, top-k);
2. the pack's magic decides the reader: a TargetPack needs ``target_policy_id``, an ExpertPack must not have one;
   the reader checks the model identity and manifest hash, and the pack must hold every routed-expert tensor;
3. the model is created on the ``meta`` device, every ``mlp`` is replaced by this package's block (router kept, for
   Qwen also the shared expert and its gate), then materialised empty on the target device, so the BF16 expert
   tensors never exist;
4. the dense tensors are read shard by shard from the Safetensors files named by ``model.safetensors.index.json``;
   the names the index lists for routed experts are counted and skipped, and the dense set must equal the model's
   ``state_dict`` exactly;
5. the rotary tables, which are not part of ``state_dict``, are rebuilt.

``expected_layers`` (not in the reference, where the depth is fixed) admits a checkpoint of the same layer shapes
with fewer layers: the pack's policy still names all layers of the full model, but only the first
``expected_layers`` need their tensors.  The parity test of the host uses it so that a CPU run of the reference on
the same files takes seconds.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Optional

import torch

from . import custom_op, native_backend
from .blocks import QuantizedMoEBlock, QuantizedQwenMoEBlock
from .formats import ContractError
from .pack_files import ExpertPackFile, NativeExpertPackFile, NativeTargetPackFile, TargetPackFile

_EXPERT_TENSOR = re.compile(r"^model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


@dataclass(frozen=True)
class FixedModel:
    """Identity and shapes of one of the two models the reference is fixed to (``src/uma_qmoe/fixed_models.py``)."""

    label: str
    model_id: str
    model_revision: str
    model_type: str
    layers: int
    experts: int
    top_k: int
    hidden: int
    intermediate: int


OLMOE = FixedModel("OLMoE", "allenai/OLMoE-1B-7B-0125", "9b0c1aa87e34a20052389dce1f0cf01da783f654", "olmoe",
                   16, 64, 8, 2048, 1024)
QWEN1_5_MOE = FixedModel("Qwen", "Qwen/Qwen1.5-MoE-A2.7B", "1a758c50ecb6350748b9ce0a99d2352fd9fc11c9", "qwen2_moe",
                         24, 60, 4, 2048, 1408)


@dataclass
class FixedHost:
    model: Any
    expert_pack: Any
    pack_handle: int
    evidence: dict[str, Any]

    def close(self) -> None:
        custom_op.unregister_expert_pack(self.pack_handle)       # drains calls in flight, drops the device copies
        self.expert_pack.close()

    def __enter__(self) -> "FixedHost":
        return self

    def __exit__(self, *_: Any) -> None:
        self.close()


FixedOlmoeHost = FixedHost
FixedQwenHost = FixedHost


def is_expert_tensor_name(name: str) -> bool:
    return _EXPERT_TENSOR.fullmatch(name) is not None


def _open_pack(spec: FixedModel, path: Path, manifest: str, policy_id: Optional[str], native: bool):
    try:
        with path.open("rb") as stream:
            magic = stream.read(8)
    except OSError as exc:
        raise ContractError(f"cannot read compressed {spec.label} pack {path}: {exc}") from exc
    identity = dict(expected_model_id=spec.model_id, expected_model_revision=spec.model_revision,
                    expected_model_manifest_sha256=manifest)
    if magic == TargetPackFile.MAGIC:
        if not policy_id:
            raise ContractError(f"{spec.label} TargetPack loading requires a policy id")
        return (NativeTargetPackFile if native else TargetPackFile)(path, expected_policy_id=policy_id, **identity)
    if policy_id is not None:
        raise ContractError(f"{spec.label} ExpertPack cannot satisfy a TargetPack policy id")
    return (NativeExpertPackFile if native else ExpertPackFile)(path, **identity)


def _require_every_expert(spec: FixedModel, reader: Any, layers: int) -> None:
    want = {f"model.layers.{l}.mlp.experts.{e}.{p}.weight": ((spec.hidden, spec.intermediate) if p == "down_proj"
                                                              else (spec.intermediate, spec.hidden))
            for l in range(layers) for e in range(spec.experts) for p in ("gate_proj", "up_proj", "down_proj")}
    have = {name: shape for name, shape in reader.shapes().items()
            if layers == spec.layers or ((m := _EXPERT_TENSOR.fullmatch(name)) is not None and int(m.group(1)) < layers)}
    if have != want:
        missing = sorted(set(want) - set(have))
        unexpected = sorted(set(have) - set(want))
        wrong = sorted(n for n in set(have) & set(want) if have[n] != want[n])
        raise ContractError(f"fixed {spec.label} tensor set mismatch: missing={missing[:8]!r}, "
                            f"unexpected={unexpected[:8]!r}, wrong_shape={wrong[:8]!r}")


def _rebuild_rotary(model: Any, config: Any, device: str) -> None:
    """``to_empty`` leaves the rotary frequency tables, which no checkpoint stores, uninitialised."""
    model.model.rotary_emb = type(model.model.rotary_emb)(config).to(device=device)
    stored = set(model.state_dict())
    loose = {name: buf for name, buf in model.named_buffers() if name not in stored}
    if set(loose) != {"model.rotary_emb.inv_freq", "model.rotary_emb.original_inv_freq"}:
        raise ContractError(f"unexpected buffers outside the checkpoint: {sorted(loose)!r}")
    for name, buf in loose.items():
        if buf.is_meta or not bool(torch.isfinite(buf).all()):
            raise ContractError(f"buffer {name!r} is not initialised")


def _attribute(root: Any, dotted: str) -> tuple[Any, str]:
    *path, leaf = dotted.split(".")
    node = root
    for part in path:
        node = node[int(part)] if part.isdigit() else getattr(node, part)
    return node, leaf


def _load_dense(spec: FixedModel, model: Any, root: Path, device: str, layers: int) -> tuple[int, int, int]:
    from safetensors import safe_open

    try:
        weight_map = json.loads((root / "model.safetensors.index.json").read_text(encoding="utf-8"))["weight_map"]
    except (OSError, json.JSONDecodeError, KeyError) as exc:
        raise ContractError(f"cannot load fixed {spec.label} Safetensors index") from exc
    if not isinstance(weight_map, dict):
        raise ContractError(f"fixed {spec.label} weight_map must be an object")
    needed = set(model.state_dict())
    shards: dict[str, list[str]] = {}
    skipped = 0
    listed = set()
    for name, shard in weight_map.items():
        if not isinstance(name, str) or not isinstance(shard, str) or not shard:
            raise ContractError(f"fixed {spec.label} weight_map entries must be strings")
        if is_expert_tensor_name(name):
            skipped += 1                                   # never opened: the pack holds these
            continue
        listed.add(name)
        shards.setdefault(shard, []).append(name)
    if listed != needed:
        raise ContractError(f"fixed {spec.label} dense checkpoint set mismatch: missing={sorted(needed - listed)[:8]!r}, "
                            f"unexpected={sorted(listed - needed)[:8]!r}")
    count = nbytes = 0
    with torch.no_grad():
        for shard in sorted(shards):
            with safe_open(root / shard, framework="pt", device="cpu") as source:
                for name in sorted(shards[shard]):
                    value = source.get_tensor(name)
                    if value.dtype != torch.bfloat16:
                        raise ContractError(f"dense tensor {name!r} is not BF16")
                    parent, leaf = _attribute(model, name)
                    target = getattr(parent, leaf)
                    if tuple(target.shape) != tuple(value.shape):
                        raise ContractError(f"dense tensor {name!r} shape mismatch")
                    target.copy_(value.to(device=device))
                    count += 1
                    nbytes += value.numel() * value.element_size()
    if skipped != layers * spec.experts * 3:
        raise ContractError(f"expected to skip {layers * spec.experts * 3} {spec.label} expert tensors, skipped {skipped}")
    return count, nbytes, skipped


def _load_fixed(spec: FixedModel, model_directory: str | Path, expert_pack_path: str | Path, *, model_manifest_sha256: str,
                device: str, performance_mode: bool, target_policy_id: Optional[str], expected_layers: Optional[int],
                native_reader: bool) -> FixedHost:
    from transformers import AutoConfig, AutoModelForCausalLM

    root, pack_path = Path(model_directory), Path(expert_pack_path)
    layers = spec.layers if expected_layers is None else int(expected_layers)
    if not 1 <= layers <= spec.layers:
        raise ContractError(f"expected_layers must be in [1, {spec.layers}]")
    config = AutoConfig.from_pretrained(root, local_files_only=True, trust_remote_code=False)
    observed = (getattr(config, "model_type", None), getattr(config, "num_hidden_layers", None),
                getattr(config, "num_experts", None), getattr(config, "num_experts_per_tok", None))
    if observed != (spec.model_type, layers, spec.experts, spec.top_k):
        raise ContractError(f"unexpected fixed {spec.label} architecture {observed!r}")
    reader = _open_pack(spec, pack_path, model_manifest_sha256, target_policy_id, native_reader)
    try:
        _require_every_expert(spec, reader, layers)
        native_backend.install_mixed_target_backend() if performance_mode else custom_op.register_moe_forward()
        handle = custom_op.register_expert_pack(reader)
    except BaseException:
        reader.close()
        raise
    try:
        with torch.device("meta"):
            model = AutoModelForCausalLM.from_config(config, dtype=torch.bfloat16, trust_remote_code=False)
        for index, layer in enumerate(model.model.layers):
            old = layer.mlp
            if spec is QWEN1_5_MOE:
                layer.mlp = QuantizedQwenMoEBlock(old.gate, old.shared_expert, old.shared_expert_gate, layer_index=index,
                                                  pack_handle=handle, performance_mode=performance_mode)
            else:
                layer.mlp = QuantizedMoEBlock(old.gate, layer_index=index, pack_handle=handle,
                                              performance_mode=performance_mode)
        model.to_empty(device=device)
        _rebuild_rotary(model, config, device)
        dense_count, dense_bytes, skipped = _load_dense(spec, model, root, device, layers)
        if any(".mlp.experts." in name for name, _ in model.named_parameters()):
            raise ContractError(f"compressed {spec.label} host still contains expert Parameters")
        if any(t.is_meta for t in (*model.parameters(), *model.buffers())):
            raise ContractError(f"compressed {spec.label} host contains meta tensors")
        model.eval()
        blocks = sum(isinstance(layer.mlp, (QuantizedMoEBlock, QuantizedQwenMoEBlock)) for layer in model.model.layers)
        if blocks != layers:
            raise ContractError(f"compressed {spec.label} host did not replace every MoE block")
        if reader.mapping_count != 1:
            raise ContractError(f"compressed {spec.label} host mapped its pack more than once")
        evidence = {
            "model_id": spec.model_id, "model_revision": spec.model_revision, "device": device,
            "performance_mode": performance_mode, "dense_tensor_count": dense_count, "dense_tensor_bytes": dense_bytes,
            "skipped_expert_tensor_count": skipped, "loaded_expert_tensor_count": 0, "expert_parameter_count": 0,
            "quantized_moe_block_count": blocks,
            "model_parameter_bytes": sum(p.numel() * p.element_size() for p in model.parameters()),
            "expert_pack_size_bytes": pack_path.stat().st_size, "expert_pack_mapping_count": reader.mapping_count,
            "torch_allocated_bytes": int(torch.cuda.memory_allocated(device)) if str(device).startswith("cuda") else 0,
            "torch_reserved_bytes": int(torch.cuda.memory_reserved(device)) if str(device).startswith("cuda") else 0,
        }
        return FixedHost(model, reader, handle, evidence)
    except BaseException:
        custom_op.unregister_expert_pack(handle)
        reader.close()
        raise


def load_fixed_qwen(model_directory: str | Path, expert_pack_path: str | Path, *, model_manifest_sha256: str,
                    device: str = "cuda:0", performance_mode: bool = False, target_policy_id: Optional[str] = None,
                    expected_layers: Optional[int] = None, native_reader: bool = True) -> FixedHost:
    """Dense Qwen1.5-MoE BF16 tensors plus one pack mapping; the routed experts run through ``torch.ops.uma_qmoe``.
    ``native_reader``: open the pack with the library's C++ reader (layers are then staged asynchronously) instead of
    the Python one; both apply the same checks."""
    return _load_fixed(QWEN1_5_MOE, model_directory, expert_pack_path, model_manifest_sha256=model_manifest_sha256,
                       device=device, performance_mode=performance_mode, target_policy_id=target_policy_id,
                       expected_layers=expected_layers, native_reader=native_reader)


def load_fixed_olmoe(model_directory: str | Path, expert_pack_path: str | Path, *, model_manifest_sha256: str,
                     device: str = "cuda:0", performance_mode: bool = False, target_policy_id: Optional[str] = None,
                     expected_layers: Optional[int] = None, native_reader: bool = True) -> FixedHost:
    """Dense OLMoE BF16 tensors plus one pack mapping."""
    return _load_fixed(OLMOE, model_directory, expert_pack_path, model_manifest_sha256=model_manifest_sha256,
                       device=device, performance_mode=performance_mode, target_policy_id=target_policy_id,
                       expected_layers=expected_layers, native_reader=native_reader)


__all__ = ["FixedHost", "FixedOlmoeHost", "FixedQwenHost", "OLMOE", "QWEN1_5_MOE", "is_expert_tensor_name",
           "load_fixed_olmoe", "load_fixed_qwen"]
