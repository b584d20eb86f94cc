"""Thin torch-facing wrappers over the C ABI: they check shapes and dtypes (the
job ``TORCH_CHECK`` does in the reference's
``src/uma_qmoe/native/packed_q4_binding.cpp:12-58,137-160,208-253``), pass raw
device pointers and the current stream, and never compute anything themselves.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _native
from .formats import ENC_BF16, ENC_Q4, ENC_Q8, ENCODING_ID


@dataclass
class DeviceLayer:
    """One staged layer: every expert's canonical bytes concatenated per projection."""

    encoding: str
    num_experts: int
    hidden: int
    intermediate: int
    gate: torch.Tensor
    up: torch.Tensor
    down: torch.Tensor
    gate_scales: Optional[torch.Tensor] = None
    up_scales: Optional[torch.Tensor] = None
    down_scales: Optional[torch.Tensor] = None

    @property
    def tensors(self) -> tuple[torch.Tensor, ...]:
        return tuple(t for t in (self.gate, self.gate_scales, self.up, self.up_scales, self.down,
                                 self.down_scales) if t is not None)

    @property
    def device_storage_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors)

    def struct(self) -> _native.Layer:
        ptr = lambda t: None if t is None else t.data_ptr()
        return _native.Layer(ptr(self.gate), ptr(self.up), ptr(self.down), ptr(self.gate_scales),
                             ptr(self.up_scales), ptr(self.down_scales), ENCODING_ID[self.encoding],
                             self.num_experts, self.hidden, self.intermediate)


@dataclass
class DeviceSharedExpert:
    gate: torch.Tensor      # [S, H] bf16
    up: torch.Tensor        # [S, H] bf16
    down: torch.Tensor      # [H, S] bf16
    gate_vec: torch.Tensor  # [H] or [1, H] bf16

    def struct(self) -> _native.SharedExpert:
        return _native.SharedExpert(self.gate.data_ptr(), self.up.data_ptr(), self.down.data_ptr(),
                                    self.gate_vec.data_ptr(), int(self.gate.shape[0]))


def _stream(device: torch.device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda_bf16(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor; there is no CPU path")
    if t.dtype != torch.bfloat16:
        raise RuntimeError(f"{what} must be BF16")
    if not t.is_contiguous():
        raise RuntimeError(f"{what} must be contiguous")


def decode_workspace(layer: DeviceLayer, top_k: int, shared: Optional[DeviceSharedExpert],
                     device: torch.device) -> torch.Tensor:
    """Zeroed workspace for :func:`moe_decode` (one per stream of calls)."""
    s_inter = int(shared.gate.shape[0]) if shared is not None else 0
    n = _native.lib().umaq_decode_workspace_bytes(top_k, layer.intermediate, s_inter)
    return torch.zeros((n + 255) // 256 * 256, dtype=torch.uint8, device=device)


def moe_decode(layer: DeviceLayer, hidden: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
               workspace: torch.Tensor, shared: Optional[DeviceSharedExpert] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token through the routed experts (and the Qwen shared expert)."""
    _require_cuda_bf16(hidden, "hidden_states")
    if hidden.numel() != layer.hidden:
        raise RuntimeError(f"decode path takes exactly one token of hidden size {layer.hidden}")
    top_k = indices.numel()
    if indices.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("expert_indices must use int32 or int64")
    if weights.dtype != torch.float32 or weights.numel() != top_k:
        raise RuntimeError("routing_weights must be float32 with one weight per route")
    if not (indices.is_contiguous() and weights.is_contiguous()):
        raise RuntimeError("routes must be contiguous")
    if out is None:
        out = torch.empty_like(hidden)
    code = _native.lib().umaq_moe_decode(
        C.byref(layer.struct()), C.byref(shared.struct()) if shared is not None else None,
        hidden.data_ptr(), indices.data_ptr(), int(indices.dtype == torch.int64), weights.data_ptr(), top_k,
        out.data_ptr(), workspace.data_ptr(), workspace.numel(), _stream(hidden.device))
    _native.check(code, "umaq_moe_decode")
    return out


def prefill_workspace(layer: DeviceLayer, tokens: int, top_k: int, shared: Optional[DeviceSharedExpert],
                      device: torch.device) -> torch.Tensor:
    s_inter = int(shared.gate.shape[0]) if shared is not None else 0
    n = _native.lib().umaq_prefill_workspace_bytes(tokens, top_k, layer.num_experts, layer.hidden,
                                                   layer.intermediate, s_inter)
    ws = torch.empty((n + 255) // 256 * 256, dtype=torch.uint8, device=device)
    ws[:256].zero_()
    return ws


def moe_prefill(layer: DeviceLayer, hidden: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                workspace: torch.Tensor, shared: Optional[DeviceSharedExpert] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[tokens, H] through the routed experts (and the Qwen shared expert) on the tensor cores."""
    _require_cuda_bf16(hidden, "hidden_states")
    flat = hidden.reshape(-1, hidden.shape[-1])
    tokens = flat.shape[0]
    if flat.shape[1] != layer.hidden:
        raise RuntimeError(f"hidden size must be {layer.hidden}")
    if indices.dtype not in (torch.int32, torch.int64) or indices.ndim != 2 or indices.shape[0] != tokens:
        raise RuntimeError("expert_indices must be [tokens, top_k] int32 or int64")
    if weights.dtype != torch.float32 or weights.shape != indices.shape:
        raise RuntimeError("routing_weights must be float32 with the shape of expert_indices")
    if not (indices.is_contiguous() and weights.is_contiguous()):
        raise RuntimeError("routes must be contiguous")
    if out is None:
        out = torch.empty_like(flat)
    code = _native.lib().umaq_moe_prefill(
        C.byref(layer.struct()), C.byref(shared.struct()) if shared is not None else None, flat.data_ptr(),
        indices.data_ptr(), int(indices.dtype == torch.int64), weights.data_ptr(), tokens, indices.shape[1],
        out.data_ptr(), workspace.data_ptr(), workspace.numel(), _stream(hidden.device))
    _native.check(code, "umaq_moe_prefill")
    return out.reshape(hidden.shape)


def prefill_status(workspace: torch.Tensor) -> int:
    return int(workspace[0:4].view(torch.int32).item())


def route_topk(hidden: torch.Tensor, router_weight: torch.Tensor, top_k: int, renormalize: bool,
               return_logits: bool = False):
    """Fused router: (weights [T,k] f32, indices [T,k] i64[, logits [T,E] bf16])."""
    _require_cuda_bf16(hidden, "hidden_states")
    _require_cuda_bf16(router_weight, "router weight")
    flat = hidden.reshape(-1, hidden.shape[-1])
    tokens, experts = flat.shape[0], router_weight.shape[0]
    w = torch.empty((tokens, top_k), dtype=torch.float32, device=hidden.device)
    idx = torch.empty((tokens, top_k), dtype=torch.int64, device=hidden.device)
    logits = torch.empty((tokens, experts), dtype=torch.bfloat16, device=hidden.device) if return_logits else None
    code = _native.lib().umaq_route_topk(flat.data_ptr(), router_weight.data_ptr(), tokens, flat.shape[1], experts,
                                         top_k, int(renormalize), w.data_ptr(), idx.data_ptr(),
                                         logits.data_ptr() if logits is not None else None, _stream(hidden.device))
    _native.check(code, "umaq_route_topk")
    return (w, idx, logits) if return_logits else (w, idx)


@dataclass
class SortedRoutes:
    """Device-side result of :func:`route_sort`."""

    counts: torch.Tensor          # [E] int32
    offsets: torch.Tensor         # [E + 1] int32
    sorted_route: torch.Tensor    # [routes] int32: route ids (token * top_k + slot) in expert order
    route_pos: torch.Tensor       # [routes] int32: position of each route in that order
    sorted_weight: torch.Tensor   # [routes] float32
    num_tiles: torch.Tensor       # [1] int32
    tile_table: torch.Tensor      # [3 * max_tiles] int32
    max_tiles: int
    status: torch.Tensor          # [1] uint32 as int32


def route_sort(indices: torch.Tensor, weights: torch.Tensor, num_experts: int) -> SortedRoutes:
    """Stable sort of the routes by expert, with the grouped GEMM's tile list."""
    if not indices.is_cuda or indices.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("expert_indices must be a CUDA int32 or int64 tensor")
    if weights.dtype != torch.float32 or weights.shape != indices.shape:
        raise RuntimeError("routing_weights must be float32 with the shape of expert_indices")
    tokens, top_k = indices.shape
    routes = tokens * top_k
    dev = indices.device
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=dev)
    max_tiles = (routes + 127) // 128 + num_experts
    scratch = i32(((routes + 2047) // 2048) * num_experts)
    r = SortedRoutes(i32(num_experts), i32(num_experts + 1), i32(routes), i32(routes),
                     torch.empty(routes, dtype=torch.float32, device=dev), i32(1), i32(3 * max_tiles), max_tiles,
                     torch.zeros(1, dtype=torch.int32, device=dev))
    code = _native.lib().umaq_route_sort(
        indices.contiguous().data_ptr(), int(indices.dtype == torch.int64), weights.contiguous().data_ptr(), tokens,
        top_k, num_experts, r.counts.data_ptr(), r.offsets.data_ptr(), r.sorted_route.data_ptr(),
        r.route_pos.data_ptr(), r.sorted_weight.data_ptr(), r.num_tiles.data_ptr(), r.tile_table.data_ptr(),
        max_tiles, r.status.data_ptr(), scratch.data_ptr(), scratch.numel(), _stream(dev))
    _native.check(code, "umaq_route_sort")
    return r


def gather_rows(hidden: torch.Tensor, sorted_route: Optional[torch.Tensor], top_k: int, permute: bool) -> torch.Tensor:
    _require_cuda_bf16(hidden, "hidden_states")
    routes = sorted_route.numel() if sorted_route is not None else hidden.shape[0]
    out = torch.empty((routes, hidden.shape[1]), dtype=torch.bfloat16, device=hidden.device)
    code = _native.lib().umaq_gather_rows(hidden.data_ptr(), sorted_route.data_ptr() if sorted_route is not None else None,
                                          top_k, routes, hidden.shape[1], int(permute), out.data_ptr(),
                                          _stream(hidden.device))
    _native.check(code, "umaq_gather_rows")
    return out


def grouped_gemm(layer: DeviceLayer, mode: int, act: torch.Tensor, routes: SortedRoutes,
                 route_weight: Optional[torch.Tensor] = None, permute_out: bool = False,
                 out: Optional[torch.Tensor] = None, variant: int = 0) -> torch.Tensor:
    """One grouped GEMM launch (mode 0: gate/up + SwiGLU, mode 1: down * routing weight).
    ``variant``: 0/1 the default one-CTA-per-tile kernel, 2 the CTA-pair (cta_group::2) kernel."""
    _require_cuda_bf16(act, "activations")
    n = layer.intermediate if mode == 0 else layer.hidden
    if out is None:
        out = torch.empty((act.shape[0], n), dtype=torch.bfloat16, device=act.device)
    code = _native.lib().umaq_grouped_gemm(
        C.byref(layer.struct()), mode, act.data_ptr(), act.shape[0], routes.num_tiles.data_ptr(),
        routes.tile_table.data_ptr(), routes.max_tiles, route_weight.data_ptr() if route_weight is not None else None,
        int(permute_out), out.data_ptr(), routes.status.data_ptr(), variant, _stream(act.device))
    _native.check(code, "umaq_grouped_gemm")
    return out


def grouped_gemm_by_index(layer: DeviceLayer, hidden: torch.Tensor, routes: SortedRoutes, top_k: int,
                          permute_out: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The gate/up GEMM fetching its activation rows by index from ``hidden`` ([tokens, H]; permuted k order for a
    quantised layer), as ``moe_prefill`` runs it: no ``[routes, H]`` copy of the activations."""
    _require_cuda_bf16(hidden, "hidden_states")
    n_routes = routes.sorted_route.numel()
    if out is None:
        out = torch.empty((n_routes, layer.intermediate), dtype=torch.bfloat16, device=hidden.device)
    code = _native.lib().umaq_grouped_gemm_by_index(
        C.byref(layer.struct()), hidden.data_ptr(), routes.sorted_route.data_ptr(), top_k, n_routes,
        routes.num_tiles.data_ptr(), routes.tile_table.data_ptr(), routes.max_tiles, int(permute_out), out.data_ptr(),
        routes.status.data_ptr(), _stream(hidden.device))
    _native.check(code, "umaq_grouped_gemm_by_index")
    return out


def ep_local_ids(indices: torch.Tensor, ranks: int, rank: int, experts_per_rank: int, interleaved: bool) -> torch.Tensor:
    """int32 local expert ids of the routes this rank owns, -1 elsewhere (see ``umaq_ep_local_ids``)."""
    if not indices.is_cuda or indices.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("expert_indices must be a CUDA int32 or int64 tensor")
    idx = indices.contiguous()
    out = torch.empty(idx.shape, dtype=torch.int32, device=idx.device)
    code = _native.lib().umaq_ep_local_ids(idx.data_ptr(), int(idx.dtype == torch.int64), idx.numel(), ranks, rank,
                                           experts_per_rank, 0 if interleaved else 1, out.data_ptr(), _stream(idx.device))
    _native.check(code, "umaq_ep_local_ids")
    return out


def ep_pack(hidden: torch.Tensor, routes: SortedRoutes, sorted_key: torch.Tensor, top_k: int, ranks: int,
            experts_per_rank: int, capacity: int, send_rows: torch.Tensor, send_meta: torch.Tensor,
            overflow: torch.Tensor) -> torch.Tensor:
    """Fixed-capacity expert-parallel dispatch (see ``umaq_ep_pack``); returns the slot of every route."""
    _require_cuda_bf16(hidden, "hidden_states")
    n = routes.sorted_route.numel()
    if sorted_key.dtype != torch.int32 or sorted_key.numel() != n:
        raise RuntimeError("sorted_key must be int32 with one entry per route")
    if send_rows.shape != (ranks * capacity, hidden.shape[1]) or send_meta.shape != (ranks * capacity, 2):
        raise RuntimeError("send buffers must hold ranks * capacity slots")
    route_slot = torch.empty(n, dtype=torch.int32, device=hidden.device)
    code = _native.lib().umaq_ep_pack(
        hidden.data_ptr(), routes.sorted_route.data_ptr(), sorted_key.data_ptr(), routes.sorted_weight.data_ptr(),
        routes.offsets.data_ptr(), n, top_k, hidden.shape[1], ranks, experts_per_rank, capacity, send_rows.data_ptr(),
        send_meta.data_ptr(), route_slot.data_ptr(), overflow.data_ptr(), _stream(hidden.device))
    _native.check(code, "umaq_ep_pack")
    return route_slot


def ep_peers(pointers: list[int], rank: int) -> _native.EpPeers:
    """Table of the ranks' exchange buffers as seen from this process (see ``umaq_ep_peers``)."""
    if not 1 <= len(pointers) <= 8 or not 0 <= rank < len(pointers):
        raise RuntimeError("between 1 and 8 ranks, and a rank inside that range")
    table = _native.EpPeers()
    for i, ptr in enumerate(pointers):
        table.base[i] = ptr
    table.ranks, table.rank = len(pointers), rank
    return table


EP_LOCAL_IDS, EP_K_PERMUTED = 1, 2          # flags of umaq_ep_push


def ep_push(hidden: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, experts_per_rank: int, interleaved: bool,
            peers: _native.EpPeers, rows_offset: int, ids_offset: int, weights_offset: int, present: torch.Tensor,
            flags: int = 0) -> None:
    """Rows and routes of the local tokens into every rank's buffer (see ``umaq_ep_push``).  ``flags``:
    ``EP_LOCAL_IDS`` = the ids arrive local to their destination (-1 for other ranks' routes), ``EP_K_PERMUTED`` =
    the rows arrive in the k order of the quantised GEMMs."""
    _require_cuda_bf16(hidden, "hidden_states")
    tokens, top_k = indices.shape
    if weights.dtype != torch.float32 or weights.shape != indices.shape or indices.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("routes must be int32/int64 indices and float32 weights of one shape")
    if present.dtype != torch.int32 or present.numel() != tokens * peers.ranks:
        raise RuntimeError("present must be int32 [tokens, ranks]")
    code = _native.lib().umaq_ep_push(hidden.data_ptr(), indices.contiguous().data_ptr(), int(indices.dtype == torch.int64),
                                      weights.contiguous().data_ptr(), tokens, top_k, hidden.shape[1], experts_per_rank,
                                      0 if interleaved else 1, flags, C.byref(peers), rows_offset, ids_offset, weights_offset,
                                      present.data_ptr(), _stream(hidden.device))
    _native.check(code, "umaq_ep_push")


def ep_barrier(peers: _native.EpPeers, flags_offset: int, epoch: torch.Tensor, status: torch.Tensor) -> None:
    """Barrier across the ranks' streams (bounded device-side wait; see ``umaq_ep_barrier``)."""
    code = _native.lib().umaq_ep_barrier(C.byref(peers), flags_offset, epoch.data_ptr(), status.data_ptr(),
                                         _stream(epoch.device))
    _native.check(code, "umaq_ep_barrier")


def moe_prefill_to_peers(layer: DeviceLayer, hidden: torch.Tensor, local_indices: torch.Tensor, weights: torch.Tensor,
                         peers: _native.EpPeers, parts_offset: int, segment_rows: int, workspace: torch.Tensor,
                         rows_k_permuted: bool = False) -> None:
    """This rank's experts over the pushed rows of all ranks, partial sums written into the owners' buffers."""
    _require_cuda_bf16(hidden, "hidden_states")
    tokens, top_k = local_indices.shape
    code = _native.lib().umaq_moe_prefill_to_peers(
        C.byref(layer.struct()), hidden.data_ptr(), local_indices.data_ptr(), int(local_indices.dtype == torch.int64),
        weights.data_ptr(), tokens, top_k, C.byref(peers), parts_offset, segment_rows, int(rows_k_permuted), workspace.data_ptr(),
        workspace.numel(), _stream(hidden.device))
    _native.check(code, "umaq_moe_prefill_to_peers")


def ep_layer(layer: DeviceLayer, hidden: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, experts_per_rank: int,
             interleaved: bool, ex, workspace: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One expert-parallel layer over the local tokens through the peer-memory exchange ``ex`` (a
    :class:`uma_qmoe_b200.ep.PeerExchange`): push, barrier, local experts with the combine writing to the owners,
    barrier, final combine — all issued by one native call (``umaq_ep_layer``)."""
    _require_cuda_bf16(hidden, "hidden_states")
    tokens, top_k = indices.shape
    if weights.dtype != torch.float32 or weights.shape != indices.shape or indices.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("routes must be int32/int64 indices and float32 weights of one shape")
    if tokens != ex.tokens or not hidden.is_contiguous() or not indices.is_contiguous() or not weights.is_contiguous():
        raise RuntimeError("ep_layer takes contiguous tensors of the exchange's token count")
    if out is None:
        out = torch.empty_like(hidden)
    code = _native.lib().umaq_ep_layer(
        C.byref(layer.struct()), hidden.data_ptr(), indices.data_ptr(), int(indices.dtype == torch.int64), weights.data_ptr(),
        tokens, top_k, experts_per_rank, 0 if interleaved else 1, C.byref(ex.peers), ex.off_rows, ex.off_ids, ex.off_w,
        ex.off_parts, ex.off_flags, ex.present.data_ptr(), ex.part_pos.data_ptr(), ex.epoch.data_ptr(), ex.status.data_ptr(),
        workspace.data_ptr(), workspace.numel(), out.data_ptr(), _stream(hidden.device))
    _native.check(code, "umaq_ep_layer")
    return out


def combine_routes(weighted: torch.Tensor, indices: torch.Tensor, route_pos: torch.Tensor,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ordered BF16 top-k combine of per-route weighted outputs."""
    _require_cuda_bf16(weighted, "weighted outputs")
    tokens, top_k = indices.shape
    if out is None:
        out = torch.empty((tokens, weighted.shape[1]), dtype=torch.bfloat16, device=weighted.device)
    code = _native.lib().umaq_combine_routes(weighted.data_ptr(), indices.contiguous().data_ptr(),
                                             int(indices.dtype == torch.int64), route_pos.data_ptr(), tokens, top_k,
                                             weighted.shape[1], out.data_ptr(), _stream(weighted.device))
    _native.check(code, "umaq_combine_routes")
    return out


def probe_stream(buffer: torch.Tensor, mode: int, status: Optional[torch.Tensor] = None) -> None:
    """One launch that only reads `buffer` (measurement aid): mode 0 = 16-byte loads from many CTAs, 1 = bulk copies
    into a shared-memory ring from one CTA per SM."""
    code = _native.lib().umaq_probe_stream(buffer.data_ptr(), buffer.numel() * buffer.element_size(), mode,
                                           status.data_ptr() if status is not None else None, _stream(buffer.device))
    _native.check(code, "umaq_probe_stream")


def workspace_status(workspace: torch.Tensor) -> int:
    """Sticky device-side status word of a workspace (synchronises)."""
    return int(workspace[8:12].view(torch.int32).item())


def quantize_groups(values: torch.Tensor, encoding: str) -> tuple[torch.Tensor, torch.Tensor]:
    """Device-side packer: BF16 tensor -> (canonical codes as uint8/int8, float32 scales)."""
    _require_cuda_bf16(values, "values")
    n = values.numel()
    enc = ENCODING_ID[encoding]
    if enc == ENC_BF16:
        raise RuntimeError("bf16_le needs no quantisation")
    codes = torch.empty(n // 2 if enc == ENC_Q4 else n, dtype=torch.uint8 if enc == ENC_Q4 else torch.int8,
                        device=values.device)
    scales = torch.empty(n // 128, dtype=torch.float32, device=values.device)
    code = _native.lib().umaq_quantize_groups(values.data_ptr(), n, enc, codes.data_ptr(), scales.data_ptr(),
                                              _stream(values.device))
    _native.check(code, "umaq_quantize_groups")
    return codes, scales
