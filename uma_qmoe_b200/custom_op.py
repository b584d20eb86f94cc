"""``torch.library`` operator boundary: ``uma_qmoe::moe_forward`` and
``uma_qmoe::qwen_moe_forward`` with the reference's schemas, pack registry,
lease semantics and fail-closed dispatch, for the ``cuda_sm100`` platform.

Mirrors ``src/uma_qmoe/custom_op.py`` of the reference:

* schemas ``:591-601`` (kept verbatim), CPU/CUDA/Meta registrations ``:602-627``;
* pack registry with handles, re-entrant per-thread leases and a blocking
  ``unregister_expert_pack`` ``:51-146``;
* ``register_performance_backend`` ``:90-100`` (the platform whitelist gains
  ``cuda_sm100``; the reference's own values stay accepted);
* fail-closed dispatch ``:509-579``: with no backend registered for the observed
  platform the call raises ``performance mode has no registered <platform>
  backend; silent reference fallback is forbidden``.

What differs on purpose: this package ships only the native sm_100a
implementation.  There is no CPU implementation behind the operator, so a call
on CPU tensors, or on CUDA tensors before a backend is installed, raises -- in
either mode -- instead of running a reference path.
"""

from __future__ import annotations

import itertools
import threading
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Callable, Iterator

from .formats import ContractError

PLATFORM = "cuda_sm100"
_KNOWN_PLATFORMS = {"cpu", "cuda_sm121", "hip_gfx1151", PLATFORM}


@dataclass
class _PackState:
    reader: Any
    active_calls: int = 0
    closing: bool = False


_PACKS: dict[int, _PackState] = {}
_PACK_CONDITION = threading.Condition()
_PACK_IDS = itertools.count(1)
_PACK_LEASES = threading.local()
_LIBRARIES: list[Any] = []
_REGISTERED = False
_PERFORMANCE_BACKENDS: dict[str, Callable[..., Any]] = {}


def register_expert_pack(reader: Any) -> int:
    if getattr(reader, "mapping_count", None) != 1:
        raise ContractError("custom operator requires exactly one ExpertPack mapping")
    with _PACK_CONDITION:
        handle = next(_PACK_IDS)
        _PACKS[handle] = _PackState(reader=reader)
    return handle


def register_target_pack(reader: Any) -> int:
    """A TargetPack registers exactly like an ExpertPack (one mapping, one handle)."""
    return register_expert_pack(reader)


def _lease_counts() -> dict[int, int]:
    counts = getattr(_PACK_LEASES, "counts", None)
    if counts is None:
        counts = {}
        _PACK_LEASES.counts = counts
    return counts


def unregister_expert_pack(handle: int) -> None:
    """Close a handle: new calls are refused at once, the call returns when the
    calls in flight have drained, then every backend drops its device copies."""
    if _lease_counts().get(handle, 0):
        raise ContractError("cannot unregister an ExpertPack from its active call")
    with _PACK_CONDITION:
        state = _PACKS.get(handle)
        if state is None:
            return
        if state.closing:
            while handle in _PACKS:
                _PACK_CONDITION.wait()
            return
        state.closing = True
        while state.active_calls:
            _PACK_CONDITION.wait()
        _PACKS.pop(handle, None)
        backends = tuple(_PERFORMANCE_BACKENDS.values())
        _PACK_CONDITION.notify_all()
    for backend in backends:
        release = getattr(backend, "release_pack", None)
        if callable(release):
            release(handle)


def register_performance_backend(platform: str, implementation: Callable[..., Any]) -> None:
    """Install an explicit backend for a platform; never used as an implicit fallback."""
    if platform not in _KNOWN_PLATFORMS:
        raise ContractError(f"unsupported custom operator platform {platform!r}")
    if not callable(implementation):
        raise ContractError("custom operator backend must be callable")
    with _PACK_CONDITION:
        _PERFORMANCE_BACKENDS[platform] = implementation


@contextmanager
def acquire_expert_pack(handle: int) -> Iterator[Any]:
    """Hold one pack open across staging and asynchronous kernel submission."""
    counts = _lease_counts()
    nested = counts.get(handle, 0) > 0
    with _PACK_CONDITION:
        state = _PACKS.get(handle)
        if state is None or (state.closing and not nested):
            raise RuntimeError(f"unknown or closed ExpertPack handle {handle}")
        if not nested:
            state.active_calls += 1
        counts[handle] = counts.get(handle, 0) + 1
    try:
        yield state.reader
    finally:
        with _PACK_CONDITION:
            left = counts[handle] - 1
            if left:
                counts[handle] = left
            else:
                del counts[handle]
                state.active_calls -= 1
                _PACK_CONDITION.notify_all()


def expert_pack_for_handle(handle: int) -> Any:
    if _lease_counts().get(handle, 0) == 0:
        raise RuntimeError("ExpertPack access requires an active operator lease")
    with _PACK_CONDITION:
        state = _PACKS.get(handle)
        if state is None:
            raise RuntimeError(f"unknown or closed ExpertPack handle {handle}")
        return state.reader


def platform_of(torch: Any, hidden_states: Any) -> str:
    """``cpu`` or ``cuda_sm100``; any other device raises, as the reference's
    ``_platform`` does for devices it does not know (``custom_op.py:149-169``)."""
    kind = hidden_states.device.type
    if kind == "cpu":
        return "cpu"
    if kind != "cuda" or torch.version.hip:
        raise RuntimeError(f"uma_qmoe::moe_forward does not support {hidden_states.device}")
    capability = torch.cuda.get_device_capability(hidden_states.device)
    if capability != (10, 0):
        raise RuntimeError(f"CUDA implementation requires SM100, observed sm_{capability[0]}{capability[1]}")
    return PLATFORM


def _backend_for(platform: str) -> Any:
    with _PACK_CONDITION:
        return _PERFORMANCE_BACKENDS.get(platform)


def _dispatch(hidden_states, expert_indices, routing_weights, layer_index: int, pack_handle: int,
              performance_mode: bool = False):
    import torch

    with acquire_expert_pack(pack_handle):
        platform = platform_of(torch, hidden_states)
        backend = _backend_for(platform)
        if backend is None:
            if performance_mode:
                raise RuntimeError(f"performance mode has no registered {platform} backend; "
                                   "silent reference fallback is forbidden")
            raise RuntimeError(f"no {platform} implementation is installed and this build has no reference "
                               "path; install_packed_q4_backend() first (silent reference fallback is forbidden)")
        return backend(hidden_states, expert_indices, routing_weights, layer_index, pack_handle)


def _qwen_dispatch(hidden_states, expert_indices, routing_weights, layer_index: int, pack_handle: int,
                   performance_mode: bool = False):
    import torch

    with acquire_expert_pack(pack_handle):
        platform = platform_of(torch, hidden_states)
        qwen_forward = getattr(_backend_for(platform), "qwen_forward", None)
        if not callable(qwen_forward):
            if performance_mode:
                raise RuntimeError(f"performance mode has no Qwen-capable {platform} backend; "
                                   "silent reference fallback is forbidden")
            raise RuntimeError(f"no Qwen-capable {platform} implementation is installed and this build has no "
                               "reference path (silent reference fallback is forbidden)")
        return qwen_forward(hidden_states, expert_indices, routing_weights, layer_index, pack_handle)


_SCHEMA_ARGS = ("(Tensor hidden_states, Tensor expert_indices, Tensor routing_weights, int layer_index, "
                "int pack_handle, bool performance_mode=False) -> Tensor")


def register_moe_forward() -> None:
    """Register both operators once.  If another package already defined the
    ``uma_qmoe`` namespace in this process (the reference itself), its
    definitions are kept and the CUDA entries are replaced by this package's."""
    global _REGISTERED
    with _PACK_CONDITION:
        if _REGISTERED:
            return
        import torch

        have = hasattr(torch.ops, "uma_qmoe") and hasattr(torch.ops.uma_qmoe, "moe_forward")
        if not have:
            definition = torch.library.Library("uma_qmoe", "DEF")
            definition.define("moe_forward" + _SCHEMA_ARGS)
            definition.define("qwen_moe_forward" + _SCHEMA_ARGS)
            _LIBRARIES.append(definition)
        fresh = not have
        for key, fns in (("CPU", (_dispatch, _qwen_dispatch)), ("CUDA", (_dispatch, _qwen_dispatch))):
            if not fresh and key == "CPU":
                continue            # keep the other package's CPU path
            lib = torch.library.Library("uma_qmoe", "IMPL", key)
            lib.impl("moe_forward", fns[0], allow_override=True) if not fresh else lib.impl("moe_forward", fns[0])
            lib.impl("qwen_moe_forward", fns[1], allow_override=True) if not fresh else lib.impl("qwen_moe_forward", fns[1])
            _LIBRARIES.append(lib)
        if fresh:
            meta = torch.library.Library("uma_qmoe", "IMPL", "Meta")
            empty_like = lambda hidden_states, _i, _w, _l, _p, _m=False: hidden_states.new_empty(hidden_states.shape)
            meta.impl("moe_forward", empty_like)
            meta.impl("qwen_moe_forward", empty_like)
            _LIBRARIES.append(meta)
        _REGISTERED = True


__all__ = [
    "PLATFORM",
    "acquire_expert_pack",
    "expert_pack_for_handle",
    "platform_of",
    "register_expert_pack",
    "register_moe_forward",
    "register_performance_backend",
    "register_target_pack",
    "unregister_expert_pack",
]
