"""The sm_100a performance backend behind ``uma_qmoe::moe_forward`` /
``uma_qmoe::qwen_moe_forward``.

Same public surface as the reference's ``src/uma_qmoe/native_backend.py``
(``PackedQ4NativeBackend``, ``MixedTargetNativeBackend``,
``install_packed_q4_backend``, ``install_mixed_target_backend``,
``load_native_extension``, ``native_kernel_source_sha256``,
``observed_native_platform``; ``cache_summary()`` keys ``:457-467``;
``release_pack`` ``:469-480``), but the native side is ``libumaq_b200.so``
called through its C ABI, one fused kernel per decode call and a tcgen05
grouped-GEMM pipeline per prefill call, for every layer encoding.

Staging (``_device_layer``, reference ``:374-455`` / ``:769-956``): the first
call on a (pack handle, layer, device) copies every expert's canonical bytes,
projection by projection, through a pinned host buffer into one device tensor
per projection; nothing is dequantised, ``dequantized_weight_bytes`` stays 0.
"""

from __future__ import annotations

import threading
import warnings
from pathlib import Path
from typing import Any, Optional

from . import _native, build as _build
from .custom_op import PLATFORM, acquire_expert_pack, register_moe_forward, register_performance_backend
from .formats import ContractError, row_bytes
from .packs import expert_tensor_name

_MODELS = {
    # op name -> (layers, experts, top_k, hidden, intermediate)    src/uma_qmoe/fixed_models.py:32-55
    "olmoe": (16, 64, 8, 2048, 1024),
    "qwen": (24, 60, 4, 2048, 1408),
}


def native_kernel_source_sha256() -> str:
    return _build.source_sha256()


def observed_native_platform(torch: Any, device: Any = 0) -> str:
    if not torch.cuda.is_available():
        raise ContractError("the native backend requires a CUDA device")
    capability = torch.cuda.get_device_capability(device)
    if torch.version.hip or capability != (10, 0):
        raise ContractError(f"the native backend requires SM100 (B200), got sm_{capability[0]}{capability[1]}")
    return PLATFORM


def load_native_extension(*, build_directory: str | Path | None = None, verbose: bool = False) -> tuple[str, Any]:
    """Build (if stale) and load ``libumaq_b200.so``; returns (platform, library).

    ``build_directory`` is accepted for signature compatibility; the library is
    always built in-tree next to its sources."""
    import torch

    platform = observed_native_platform(torch)
    _build.build(verbose=verbose)
    return platform, _native.lib()


class _LayerCache:
    def __init__(self) -> None:
        self.layers: dict[tuple[int, int, str], Any] = {}
        self.lock = threading.Lock()


class _Workspace:
    """A kernel workspace owned by one (shape, device, stream) and the host's view of its sticky status word.

    After every call the first 16 bytes of the workspace (prefill status in word 0, decode status in word 2) are
    copied to pinned host memory on the call's stream and an event is recorded; the next call on this workspace,
    `cache_summary()` and `release_pack()` look at the copy once the event has completed.  Nothing on the hot
    path waits for the device."""

    __slots__ = ("kind", "buffer", "host", "event", "tokens")

    def __init__(self, kind: str, buffer: Any, tokens: int) -> None:
        import torch

        self.kind, self.buffer, self.tokens = kind, buffer, tokens
        self.host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.event: Any = None

    def publish(self, stream: Any) -> None:
        import torch

        if torch.cuda.is_current_stream_capturing():
            return                                   # a captured call reports through the workspace only
        self.host.copy_(self.buffer[:16].view(torch.int32), non_blocking=True)
        if self.event is None:
            self.event = torch.cuda.Event()
        self.event.record(stream)

    def raise_if_failed(self, wait: bool) -> None:
        import torch

        if self.event is None or torch.cuda.is_current_stream_capturing():
            return
        if wait:
            self.event.synchronize()
        elif not self.event.query():
            return
        code = int(self.host[0 if self.kind == "prefill" else 2])
        if code == 0:
            return
        # sticky on the device: clear it so that the error is reported once (all work on the buffer has finished)
        self.host.zero_()
        self.event = None
        if code == -1:                               # UMAQ_ERR_BAD_ARGUMENT: the kernels skipped a route
            self.buffer[:16].zero_()
            raise RuntimeError("expert_indices contains an invalid expert")
        self.buffer[:1024].zero_()                   # a timeout leaves stale counters behind
        raise RuntimeError(f"an earlier uma_qmoe::moe_forward call failed on the device ({_native.ERRORS.get(code, code)})")


class MixedTargetNativeBackend:
    """Executes Q4, Q8 and BF16 layers of an ExpertPack or TargetPack."""

    allowed_encodings = ("q4_group128", "q8_group128", "bf16_le")

    def __init__(self, platform: str, extension: Any) -> None:
        if platform != PLATFORM:
            raise ContractError(f"unsupported native platform {platform!r}")
        for name in _native.SIGNATURES:
            if not hasattr(extension, name):
                raise ContractError(f"native library does not export {name}")
        self.platform = platform
        self.extension = extension
        self._cache = _LayerCache()
        self._workspaces: dict[tuple, _Workspace] = {}
        self._pending: dict[tuple[int, int, str], Any] = {}      # layers being staged: (DeviceLayer, wait)
        self._linear_cache: dict[tuple[int, str, str], Any] = {}  # single tensors staged for q4_linear / q8_linear
        self._workspace_lock = threading.Lock()

    # ---- construction ---------------------------------------------------------------------
    @classmethod
    def build_and_register(cls, *, build_directory: str | Path | None = None, verbose: bool = False):
        platform, extension = load_native_extension(build_directory=build_directory, verbose=verbose)
        backend = cls(platform, extension)
        register_moe_forward()
        register_performance_backend(platform, backend)
        return backend

    # ---- staging --------------------------------------------------------------------------
    @staticmethod
    def _encoding_of(reader: Any, layer_index: int) -> str:
        if hasattr(reader, "layer_encoding"):
            return reader.layer_encoding(layer_index)
        group = int(reader.header["quantization"]["group_size"])
        if group != 128:
            raise RuntimeError(f"the native backend requires group size 128, got {group}")
        return "q4_group128"

    def _device_layer(self, pack_handle: int, layer_index: int, device: Any, reader: Any, model: str):
        import torch

        from .ops import DeviceLayer

        key = (pack_handle, layer_index, str(device))
        with self._cache.lock:
            hit = self._cache.layers.get(key)
        if hit is not None:
            return hit
        layers, experts, _k, hidden, inter = _MODELS[model]
        if not 0 <= layer_index < layers:
            name = "OLMoE" if model == "olmoe" else "Qwen"
            raise RuntimeError(f"{name} layer_index must be in [0, {layers - 1}]")
        encoding = self._encoding_of(reader, layer_index)
        if encoding not in self.allowed_encodings:
            raise RuntimeError(f"this backend cannot execute layer {layer_index} encoded as {encoding}; "
                               "install the mixed backend")
        quantised = encoding != "bf16_le"
        if hasattr(reader, "stage_layer_async"):
            # the native reader stages by itself: a worker thread, pinned chunks, copies on a stream of its own;
            # a prefetch may already be under way
            with self._cache.lock:
                pending = self._pending.pop(key, None)
            layer, wait = pending if pending is not None else self._start_staging(reader, layer_index, device, model)
            wait(torch.cuda.current_stream(device))
            with self._cache.lock:
                return self._cache.layers.setdefault(key, layer)
        staged = {}
        for proj, (rows, k) in (("gate_proj", (inter, hidden)), ("up_proj", (inter, hidden)),
                                ("down_proj", (hidden, inter))):
            nbytes = rows * row_bytes(encoding, k)
            host = torch.empty((experts, nbytes), dtype=torch.uint8).pin_memory()
            host_s = torch.empty((experts, rows * k // 128), dtype=torch.float32).pin_memory() if quantised else None
            for e in range(experts):
                data, scales, meta = reader.tensor_views(expert_tensor_name(layer_index, e, proj))
                try:
                    if tuple(meta["shape"]) != (rows, k):
                        raise RuntimeError(f"tensor {meta.get('name', proj)!r} has unexpected shape {tuple(meta['shape'])!r}")
                    if meta.get("encoding", encoding) != encoding:
                        raise RuntimeError(f"tensor of layer {layer_index} is not {encoding}")
                    if len(data) != nbytes:
                        raise RuntimeError("pack tensor byte count does not match its shape")
                    with warnings.catch_warnings():       # the mapping is read-only and is only read here
                        warnings.filterwarnings("ignore", message="The given buffer is not writable")
                        host[e].copy_(torch.frombuffer(data, dtype=torch.uint8))
                        if quantised:
                            host_s[e].copy_(torch.frombuffer(scales, dtype=torch.float32))
                finally:
                    data.release()
                    scales.release()
            staged[proj] = (host.to(device, non_blocking=True),
                            host_s.to(device, non_blocking=True) if quantised else None)
        torch.cuda.current_stream(device).synchronize()      # the pinned buffers go away after this
        layer = DeviceLayer(encoding, experts, hidden, inter, staged["gate_proj"][0], staged["up_proj"][0],
                            staged["down_proj"][0], staged["gate_proj"][1], staged["up_proj"][1],
                            staged["down_proj"][1])
        with self._cache.lock:
            return self._cache.layers.setdefault(key, layer)

    def _start_staging(self, reader: Any, layer_index: int, device: Any, model: str):
        import torch

        from .ops import DeviceLayer
        layers, experts, _k, hidden, inter = _MODELS[model]
        if not 0 <= layer_index < layers:
            raise RuntimeError(f"{'OLMoE' if model == 'olmoe' else 'Qwen'} layer_index must be in [0, {layers - 1}]")
        encoding = self._encoding_of(reader, layer_index)
        if encoding not in self.allowed_encodings:
            raise RuntimeError(f"this backend cannot execute layer {layer_index} encoded as {encoding}; "
                               "install the mixed backend")
        quantised = encoding != "bf16_le"
        codes = lambda rows, k: torch.empty(experts * rows * row_bytes(encoding, k), dtype=torch.uint8, device=device)
        scales = lambda rows, k: torch.empty(experts * rows * k // 128, dtype=torch.float32, device=device) if quantised else None
        layer = DeviceLayer(encoding, experts, hidden, inter, codes(inter, hidden), codes(inter, hidden), codes(hidden, inter),
                            scales(inter, hidden), scales(inter, hidden), scales(hidden, inter))
        # the copies run on the reader's own stream: whatever used this memory before must have finished
        torch.cuda.current_stream(device).synchronize()
        return layer, reader.stage_layer_async(layer_index, layer, device)

    def prefetch_layer(self, pack_handle: int, layer_index: int, device: Any, model: str = "olmoe") -> None:
        """Start staging a layer of a pack opened with the native reader and return at once; the first call that
        needs the layer waits for what is left.  (Nothing to do for the Python readers, which stage on demand.)"""
        import torch
        device = torch.device(device)
        key = (pack_handle, layer_index, str(device))
        with acquire_expert_pack(pack_handle) as reader:
            if not hasattr(reader, "stage_layer_async"):
                return
            with self._cache.lock:
                if key in self._cache.layers or key in self._pending:
                    return
            started = self._start_staging(reader, layer_index, device, model)
            with self._cache.lock:
                self._pending[key] = started

    def preload_layer(self, pack_handle: int, layer_index: int, device: Any, layer: Any) -> None:
        """Adopt a layer that already sits on the device in the staged layout (synthetic weights
        built with the device-side packer), instead of staging it from the pack's host bytes."""
        with self._cache.lock:
            self._cache.layers[(pack_handle, layer_index, str(device))] = layer

    def check_device_status(self) -> None:
        """Wait for the calls submitted so far and raise if one of them recorded a device-side error."""
        with self._workspace_lock:
            slots = list(self._workspaces.values())
        for slot in slots:
            slot.raise_if_failed(wait=True)

    def cache_summary(self) -> dict[str, int]:
        self.check_device_status()
        with self._cache.lock:
            layers = list(self._cache.layers.values())
        return {
            "tensor_count": sum(3 * layer.num_experts for layer in layers),
            "device_storage_bytes": sum(layer.device_storage_bytes for layer in layers),
            "dequantized_weight_bytes": 0,
        }

    def release_pack(self, pack_handle: int) -> None:
        """Drop every device copy that belongs to a closed pack handle."""
        try:
            self.check_device_status()
        finally:
            self._drop_layers(pack_handle)

    def _drop_layers(self, pack_handle: int) -> None:
        import torch
        with self._cache.lock:
            unfinished = [self._pending.pop(k) for k in [k for k in self._pending if k[0] == pack_handle]]
        for layer, wait in unfinished:              # the worker threads must be done before the mapping goes away
            wait(torch.cuda.current_stream(layer.gate.device))
        with self._cache.lock:
            for key in [k for k in self._cache.layers if k[0] == pack_handle]:
                del self._cache.layers[key]
            for key in [k for k in self._linear_cache if k[0] == pack_handle]:
                del self._linear_cache[key]

    # ---- execution ------------------------------------------------------------------------
    def _workspace(self, kind: str, layer: Any, tokens: int, top_k: int, shared: Any, device: Any, stream: Any) -> _Workspace:
        """The workspace of this shape on this stream.  Calls on different streams (or threads, which have their own
        current stream only if they set one) never share a workspace, so they may overlap on the device; a stream
        keeps one prefill workspace per layer shape, grown to the largest token count seen."""
        from . import ops

        family = (kind, str(device), int(stream.cuda_stream), layer.hidden, layer.intermediate, layer.num_experts, top_k,
                  0 if shared is None else int(shared.gate.shape[0]))
        with self._workspace_lock:
            slot = self._workspaces.get(family)
            if slot is not None and (kind == "decode" or slot.tokens >= tokens):
                return slot
        if slot is not None:
            slot.raise_if_failed(wait=True)          # the smaller buffer is about to be dropped
        if kind == "decode":
            fresh = _Workspace(kind, ops.decode_workspace(layer, top_k, shared, device), 1)
        else:
            fresh = _Workspace(kind, ops.prefill_workspace(layer, tokens, top_k, shared, device), tokens)
        with self._workspace_lock:
            self._workspaces[family] = fresh
        return fresh

    def _run(self, model: str, hidden_states: Any, expert_indices: Any, routing_weights: Any, layer_index: int,
             pack_handle: int, shared: Optional[Any] = None):
        import torch

        from . import ops

        _layers, _experts, top_k, hidden, _inter = _MODELS[model]
        label = "OLMoE" if model == "olmoe" else "Qwen"
        if hidden_states.dtype != torch.bfloat16:
            raise RuntimeError(f"{label} native backend requires BF16 hidden states")
        flat = hidden_states.reshape(-1, hidden_states.shape[-1])
        if flat.shape[-1] != hidden:
            raise RuntimeError(f"{label} native backend requires hidden size {hidden}")
        if tuple(expert_indices.shape) != (flat.shape[0], top_k):
            raise RuntimeError(f"{label} native backend requires [tokens, {top_k}] routes")
        if expert_indices.dtype not in (torch.int32, torch.int64):
            raise RuntimeError("expert_indices must use int32 or int64")
        if tuple(routing_weights.shape) != tuple(expert_indices.shape):
            raise RuntimeError("expert_indices and routing_weights shapes must match")
        with acquire_expert_pack(pack_handle) as reader:
            layer = self._device_layer(pack_handle, layer_index, hidden_states.device, reader, model)
        stream = torch.cuda.current_stream(hidden_states.device)
        for tensor in layer.tensors:
            tensor.record_stream(stream)
        flat = flat.contiguous()
        indices = expert_indices.contiguous()
        weights = routing_weights.to(dtype=torch.float32).contiguous()     # float32 routing weights, no BF16 rounding
        tokens = flat.shape[0]
        out = torch.empty_like(flat)
        if tokens == 0:                       # an empty batch has an empty result; there is nothing to launch
            return out.reshape(hidden_states.shape)
        slot = self._workspace("decode" if tokens == 1 else "prefill", layer, tokens, top_k, shared,
                               hidden_states.device, stream)
        slot.raise_if_failed(wait=False)      # an error an earlier call on this workspace left behind, if already known
        slot.buffer.record_stream(stream)
        if tokens == 1:
            ops.moe_decode(layer, flat, indices, weights, slot.buffer, shared, out=out)
        else:
            ops.moe_prefill(layer, flat, indices, weights, slot.buffer, shared, out=out)
        slot.publish(stream)
        return out.reshape(hidden_states.shape)

    # ---- one projection as a linear layer -----------------------------------------------------
    def _linear(self, input_tensor: Any, pack_handle: int, tensor_name: str, encoding: str):
        """``bf16(input . W^T)`` for one packed tensor of a registered pack (the reference backend's ``q4_linear`` /
        ``q8_linear``, ``src/uma_qmoe/native_backend.py:319-372``; there a GEMV kernel per call, here the grouped GEMM's
        down mode on a one-expert layer: rows of any count, out features a multiple of 256, in features of 128)."""
        import torch

        from . import ops
        from .ops import DeviceLayer
        if input_tensor.dtype != torch.bfloat16 or input_tensor.ndim != 2 or not input_tensor.is_cuda:
            raise RuntimeError("the native backend requires a 2-D BF16 CUDA input")
        device = input_tensor.device
        key = (pack_handle, tensor_name, str(device))
        with self._cache.lock:
            hit = self._linear_cache.get(key)
        if hit is None:
            with acquire_expert_pack(pack_handle) as reader:
                data, scales, meta = reader.tensor_views(tensor_name)
                try:
                    if meta.get("encoding", "q4_group128") != encoding:
                        raise RuntimeError(f"tensor {tensor_name!r} is not {encoding}")
                    rows, k = (int(d) for d in meta["shape"])
                    with warnings.catch_warnings():
                        warnings.filterwarnings("ignore", message="The given buffer is not writable")
                        codes = torch.frombuffer(data, dtype=torch.uint8).to(device)
                        sc = torch.frombuffer(scales, dtype=torch.float32).to(device)
                finally:
                    data.release()
                    scales.release()
            if rows % 256 or k % 128:
                raise RuntimeError(f"tensor {tensor_name!r} has a shape the linear path does not take: {(rows, k)}")
            # a one-expert layer whose "down" projection is this tensor: hidden = out features, intermediate = in
            hit = DeviceLayer(encoding, 1, rows, k, codes, codes, codes, sc, sc, sc)
            with self._cache.lock:
                hit = self._linear_cache.setdefault(key, hit)
        if input_tensor.shape[1] != hit.intermediate:
            raise RuntimeError(f"input has {input_tensor.shape[1]} features, the tensor takes {hit.intermediate}")
        n = input_tensor.shape[0]
        if n == 0:
            return input_tensor.new_empty((0, hit.hidden))
        ones = torch.ones((n, 1), dtype=torch.float32, device=device)
        routes = ops.route_sort(torch.zeros((n, 1), dtype=torch.int32, device=device), ones, 1)
        act = ops.gather_rows(input_tensor.contiguous(), None, 1, permute=True)      # the k order of the quantised GEMM
        return ops.grouped_gemm(hit, 1, act, routes, variant=1)

    def q4_linear(self, input_tensor: Any, pack_handle: int, tensor_name: str):
        return self._linear(input_tensor, pack_handle, tensor_name, "q4_group128")

    def q8_linear(self, input_tensor: Any, pack_handle: int, tensor_name: str):
        return self._linear(input_tensor, pack_handle, tensor_name, "q8_group128")

    def __call__(self, hidden_states, expert_indices, routing_weights, layer_index: int, pack_handle: int):
        return self._run("olmoe", hidden_states, expert_indices, routing_weights, layer_index, pack_handle)

    def qwen_forward(self, hidden_states, expert_indices, routing_weights, layer_index: int, pack_handle: int):
        return self._run("qwen", hidden_states, expert_indices, routing_weights, layer_index, pack_handle)

    def qwen_block_forward(self, hidden_states, expert_indices, routing_weights, layer_index: int, pack_handle: int,
                           shared: Any):
        """Routed experts plus the shared expert and its sigmoid gate in the same kernels."""
        return self._run("qwen", hidden_states, expert_indices, routing_weights, layer_index, pack_handle, shared)


class PackedQ4NativeBackend(MixedTargetNativeBackend):
    """The Q4-only backend of the reference's first milestone; other encodings are refused with the
    reference's hint to install the mixed backend (``native_backend.py:421-427``)."""

    allowed_encodings = ("q4_group128",)


def install_packed_q4_backend(*, build_directory: str | Path | None = None, verbose: bool = False):
    return PackedQ4NativeBackend.build_and_register(build_directory=build_directory, verbose=verbose)


def install_mixed_target_backend(*, build_directory: str | Path | None = None, verbose: bool = False):
    return MixedTargetNativeBackend.build_and_register(build_directory=build_directory, verbose=verbose)


__all__ = [
    "PackedQ4NativeBackend",
    "MixedTargetNativeBackend",
    "install_mixed_target_backend",
    "install_packed_q4_backend",
    "load_native_extension",
    "native_kernel_source_sha256",
    "observed_native_platform",
]
