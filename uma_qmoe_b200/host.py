"""Fixed-model host: a Hugging Face MoE model whose routed experts run on this package's kernels.

The reference builds such a host from a checkpoint and a pack file (``load_fixed_olmoe`` in
``src/uma_qmoe/compressed_loader.py:70-167``, ``load_fixed_qwen`` in ``src/uma_qmoe/qwen_compressed_loader.py:143-303``):
every ``mlp`` of a decoder layer is replaced by a block that keeps the router (and, for Qwen, the shared expert and
its gate) and sends the routed experts through ``torch.ops.uma_qmoe``.  :func:`install_quantized_blocks` does the same
swap on a model that is already on the device -- OLMoE (``gate`` + ``experts``) or Qwen2-MoE (plus ``shared_expert``
and ``shared_expert_gate``) as laid out by transformers 5.x, where the experts of a layer are two fused tensors
``gate_up_proj [E, 2I, H]`` and ``down_proj [E, H, I]``.  The experts are encoded per layer on the device
(``umaq_quantize_groups``; ``bf16_le`` layers are copied) straight into the staged layout the kernels read, adopted
by the installed back end, and the dense expert tensors are freed.

:func:`greedy_decode` is the measurement loop of the reference host (prefill, then one token per step with the
key/value cache, ``benchmarks/runners/pytorch_reference_host.py:148-164``) with CUDA-event timing.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Union

import torch

from . import custom_op, native_backend, ops
from .blocks import QuantizedMoEBlock, QuantizedQwenMoEBlock
from .formats import ContractError
from .ops import DeviceLayer


class _AdoptedWeights:
    """Pack object behind the handle of a host whose layers were encoded on the device: it only carries the
    layer policy; the tensors never exist as host bytes."""

    mapping_count = 1

    def __init__(self, encodings: Mapping[int, str]) -> None:
        self._encodings = dict(encodings)
        self.header = {"quantization": {"group_size": 128}, "policy": {"layer_encodings": {str(k): v for k, v in encodings.items()}}}

    def layer_encoding(self, layer_index: int) -> str:
        return self._encodings[layer_index]

    def tensor_views(self, name: str):
        raise ContractError(f"tensor {name!r} was encoded on the device and has no host bytes")

    def close(self) -> None:
        pass


def encode_experts(gate_up_proj: torch.Tensor, down_proj: torch.Tensor, encoding: str) -> DeviceLayer:
    """Fused HF expert tensors ``[E, 2I, H]`` / ``[E, H, I]`` (BF16, on the device) -> staged layer."""
    if gate_up_proj.dtype != torch.bfloat16 or down_proj.dtype != torch.bfloat16 or not gate_up_proj.is_cuda:
        raise RuntimeError("expert tensors must be BF16 CUDA tensors")
    experts, two_i, hidden = gate_up_proj.shape
    inter = two_i // 2
    if down_proj.shape != (experts, hidden, inter):
        raise RuntimeError(f"down_proj has shape {tuple(down_proj.shape)}, expected {(experts, hidden, inter)}")
    gate = gate_up_proj[:, :inter, :].contiguous()
    up = gate_up_proj[:, inter:, :].contiguous()
    down = down_proj.contiguous()
    if encoding == "bf16_le":
        as_bytes = lambda t: t.reshape(-1).view(torch.uint8)
        return DeviceLayer(encoding, experts, hidden, inter, as_bytes(gate), as_bytes(up), as_bytes(down), None, None, None)
    (g, gs), (u, us), (d, ds) = (ops.quantize_groups(t.reshape(-1), encoding) for t in (gate, up, down))
    return DeviceLayer(encoding, experts, hidden, inter, g, u, d, gs, us, ds)


@dataclass
class FixedModelHost:
    model: Any
    pack_handle: int
    layer_encodings: dict[int, str]
    evidence: dict[str, Any] = field(default_factory=dict)

    def close(self) -> None:
        backend = custom_op._backend_for(custom_op.PLATFORM)
        if backend is not None and hasattr(backend, "release_pack"):
            backend.release_pack(self.pack_handle)
        custom_op.unregister_expert_pack(self.pack_handle)

    def __enter__(self) -> "FixedModelHost":
        return self

    def __exit__(self, *_: Any) -> None:
        self.close()


def install_quantized_blocks(model: Any, encodings: Union[str, Mapping[int, str]], *, performance_mode: bool = True
                             ) -> FixedModelHost:
    """Replace every sparse-MoE ``mlp`` of ``model.model.layers`` and free its dense expert tensors.

    ``encodings``: one encoding for all layers or ``{layer index: encoding}`` (the TargetPack policy)."""
    layers = model.model.layers
    device = next(model.parameters()).device
    if device.type != "cuda":
        raise RuntimeError("the model must be on a CUDA device before its experts are encoded")
    sparse = [i for i, layer in enumerate(layers) if hasattr(layer.mlp, "experts") and hasattr(layer.mlp, "gate")]
    if not sparse:
        raise RuntimeError("the model has no sparse MoE layers")
    policy = {i: (encodings if isinstance(encodings, str) else encodings[i]) for i in sparse}
    backend = native_backend.install_mixed_target_backend()
    custom_op.register_moe_forward()
    handle = custom_op.register_target_pack(_AdoptedWeights(policy))
    stored = 0
    for i in sparse:
        block = layers[i].mlp
        with torch.no_grad():
            staged = encode_experts(block.experts.gate_up_proj.data, block.experts.down_proj.data, policy[i])
        backend.preload_layer(handle, i, device, staged)
        stored += staged.device_storage_bytes
        if hasattr(block, "shared_expert"):
            new = QuantizedQwenMoEBlock(block.gate, block.shared_expert, block.shared_expert_gate, layer_index=i,
                                        pack_handle=handle, performance_mode=performance_mode)
        else:
            new = QuantizedMoEBlock(block.gate, layer_index=i, pack_handle=handle, performance_mode=performance_mode)
        layers[i].mlp = new
        del block.experts, block
    torch.cuda.empty_cache()
    return FixedModelHost(model, handle, policy, {"expert_storage_bytes": stored, "sparse_layers": len(sparse),
                                                   "dequantized_weight_bytes": 0})


@torch.no_grad()
def greedy_decode(model: Any, input_ids: torch.Tensor, new_tokens: int) -> dict[str, Any]:
    """Greedy generation at batch 1: prefill, then ``new_tokens - 1`` single-token steps with the KV cache.
    Returns the generated ids, the logits of every step (float32, on the host) and device-timed TTFT / TPOT."""
    if input_ids.dim() != 2 or input_ids.shape[0] != 1 or new_tokens < 1:
        raise RuntimeError("greedy_decode takes one prompt [1, T] and at least one new token")
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(new_tokens + 1)]
    marks[0].record()
    out = model(input_ids=input_ids, use_cache=True)
    cache = out.past_key_values
    logits = [out.logits[:, -1].float()]
    token = logits[-1].argmax(dim=-1)
    tokens = [token]
    marks[1].record()
    for step in range(1, new_tokens):
        out = model(input_ids=token[:, None], past_key_values=cache, use_cache=True)
        cache = out.past_key_values
        logits.append(out.logits[:, -1].float())
        token = logits[-1].argmax(dim=-1)
        tokens.append(token)
        marks[step + 1].record()
    torch.cuda.synchronize()
    steps = [marks[i].elapsed_time(marks[i + 1]) for i in range(1, new_tokens)]
    return {"tokens": torch.cat(tokens).tolist(), "logits": torch.cat(logits).cpu(),
            "ttft_ms": marks[0].elapsed_time(marks[1]), "tpot_ms": steps}


class GraphedDecoder:
    """Batch-1 decode with the whole step -- embedding, attention over a static key/value cache, the MoE blocks,
    the LM head, the arg-max that picks the next token and the position increment -- captured once in a CUDA graph
    and replayed per token, so that the host issues one launch per token instead of a few hundred (the reference's
    host runs the step eagerly, ``benchmarks/runners/pytorch_reference_host.py:148-164``)."""

    def __init__(self, model: Any, max_len: int) -> None:
        from transformers import StaticCache

        self.model = model
        self.device = next(model.parameters()).device
        self.cache = StaticCache(config=model.config, max_cache_len=max_len)
        self.max_len = max_len
        self.token = torch.zeros((1, 1), dtype=torch.long, device=self.device)        # next input token
        self.position = torch.zeros((1,), dtype=torch.long, device=self.device)       # its position
        self.graph: Any = None
        self.logits: Any = None                                                          # logits of the last replay

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        tokens = input_ids.shape[1]
        if tokens >= self.max_len:
            raise RuntimeError("the prompt does not fit the static cache")
        self.cache.reset()
        out = self.model(input_ids=input_ids, past_key_values=self.cache,
                         cache_position=torch.arange(tokens, device=self.device), use_cache=True)
        logits = out.logits[:, -1].float()
        self.token.copy_(logits.argmax(dim=-1)[:, None])
        self.position.fill_(tokens)
        return logits

    @torch.no_grad()
    def _step(self) -> torch.Tensor:
        out = self.model(input_ids=self.token, past_key_values=self.cache, cache_position=self.position, use_cache=True)
        logits = out.logits[:, -1].float()
        self.token.copy_(logits.argmax(dim=-1)[:, None])
        self.position.add_(1)
        return logits

    def capture(self) -> None:
        """Capture one step (call after a prefill, and prefill again before generating: the two warm-up steps and
        the capture run disturb the cache state)."""
        token, position = self.token.clone(), self.position.clone()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._step()
            self._step()
            self.token.copy_(token)
            self.position.copy_(position)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                self.logits = self._step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.token.copy_(token)
        self.position.copy_(position)
        self.graph = graph

    def step(self) -> torch.Tensor:
        """One token: returns the (static) logits tensor; ``self.token`` then holds the next input."""
        if self.graph is None:
            raise RuntimeError("capture() first")
        self.graph.replay()
        return self.logits


@torch.no_grad()
def greedy_decode_graphed(model: Any, input_ids: torch.Tensor, new_tokens: int, decoder: Any = None,
                          keep_logits: bool = False) -> dict[str, Any]:
    """:func:`greedy_decode` with the decode steps replayed from a CUDA graph; the only host synchronisation is the
    one at the end."""
    if input_ids.dim() != 2 or input_ids.shape[0] != 1 or new_tokens < 1:
        raise RuntimeError("greedy_decode_graphed takes one prompt [1, T] and at least one new token")
    dec = decoder or GraphedDecoder(model, input_ids.shape[1] + new_tokens + 8)
    if dec.graph is None:
        # one-off: a throw-away prefill gives the capture a populated cache; the warm-up and capture runs leave
        # the cache and the library's host-side counters in a state that only a fresh prefill resets, so the
        # generation below always starts with its own prefill
        dec.prefill(input_ids)
        dec.capture()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(new_tokens + 1)]
    marks[0].record()
    logits = [dec.prefill(input_ids)]
    tokens = [dec.token.clone()]
    marks[1].record()
    for step in range(1, new_tokens):
        out = dec.step()
        if keep_logits:
            logits.append(out.clone())
        tokens.append(dec.token.clone())
        marks[step + 1].record()
    torch.cuda.synchronize()
    return {"tokens": torch.cat(tokens, dim=1)[0].tolist(), "logits": torch.cat(logits).cpu(),
            "ttft_ms": marks[0].elapsed_time(marks[1]),
            "tpot_ms": [marks[i].elapsed_time(marks[i + 1]) for i in range(1, new_tokens)], "decoder": dec}
