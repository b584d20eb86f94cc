"""Drop-in MoE blocks with the constructor signatures of the reference's
``QuantizedMoEBlock`` (``src/uma_qmoe/compressed_loader.py:41-67``) and
``QuantizedQwenMoEBlock`` (``src/uma_qmoe/qwen_compressed_loader.py:46-86``).

They call the same ``torch.ops.uma_qmoe`` operators; what they add is the fused path around it: the
router runs as one kernel (softmax / top-k / renormalisation), and for Qwen the shared expert, its
sigmoid gate and the final add run inside the expert kernels instead of as separate cuBLAS and
element-wise launches.
"""

from __future__ import annotations

from typing import Any

import torch

from . import ops
from .custom_op import _backend_for, platform_of
from .ops import DeviceSharedExpert


def _router_params(gate: Any) -> tuple[torch.Tensor, int, bool]:
    return gate.weight, int(gate.top_k), bool(getattr(gate, "norm_topk_prob", False))


class QuantizedMoEBlock(torch.nn.Module):
    """OLMoE router plus the compressed routed experts."""

    def __init__(self, gate: Any, *, layer_index: int, pack_handle: int, performance_mode: bool) -> None:
        super().__init__()
        self.gate = gate
        self.layer_index = layer_index
        self.pack_handle = pack_handle
        self.performance_mode = performance_mode

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        weight, top_k, renorm = _router_params(self.gate)
        flat = hidden_states.reshape(-1, hidden_states.shape[-1])
        routing_weights, selected = ops.route_topk(flat, weight, top_k, renorm)
        return torch.ops.uma_qmoe.moe_forward(hidden_states, selected, routing_weights, self.layer_index,
                                              self.pack_handle, self.performance_mode)


class QuantizedQwenMoEBlock(torch.nn.Module):
    """Qwen router, shared expert and sigmoid gate fused around the packed routed experts."""

    def __init__(self, gate: Any, shared_expert: Any, shared_expert_gate: Any, *, layer_index: int,
                 pack_handle: int, performance_mode: bool) -> None:
        super().__init__()
        self.gate = gate
        self.shared_expert = shared_expert
        self.shared_expert_gate = shared_expert_gate
        self.layer_index = layer_index
        self.pack_handle = pack_handle
        self.performance_mode = performance_mode

    def _shared(self) -> DeviceSharedExpert:
        se = self.shared_expert
        return DeviceSharedExpert(se.gate_proj.weight, se.up_proj.weight, se.down_proj.weight,
                                  self.shared_expert_gate.weight)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        batch, seq, hidden = hidden_states.shape
        flat = hidden_states.reshape(-1, hidden)
        weight, top_k, renorm = _router_params(self.gate)
        routing_weights, selected = ops.route_topk(flat, weight, top_k, renorm)
        backend = _backend_for(platform_of(torch, flat))
        fused = getattr(backend, "qwen_block_forward", None)
        if not callable(fused):
            raise RuntimeError("performance mode has no Qwen-capable backend with a fused shared expert; "
                               "silent reference fallback is forbidden")
        from .custom_op import acquire_expert_pack
        with acquire_expert_pack(self.pack_handle):
            out = fused(flat, selected, routing_weights, self.layer_index, self.pack_handle, self._shared())
        return out.reshape(batch, seq, hidden)
