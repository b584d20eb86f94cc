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
from typing import Any, Callable, Iterator

from .formats import ContractError

PLATFORM = "cuda_sm100"
_KNOWN_PLATFORMS = {"cpu", "cuda_sm121", "hip_gfx1151", PLATFORM}


class _Entry:
    """One registered pack: its reader, how many threads are inside a call on it, and whether it is being closed."""

    __slots__ = ("reader", "in_flight", "closing")

    def __init__(self, reader: Any) -> None:
        self.reader = reader
        self.in_flight = 0
        self.closing = False


class PackRegistry:
    """Handles for pack readers, leases for the calls that use them, and the installed backends.

    A lease keeps a pack open from the moment a call looks it up until its kernels are submitted.
    Leases are counted per thread, so a call may take the lease again further down (the backend
    does, to reach the reader); only a thread's outermost lease counts as a call in flight.
    Closing a handle refuses new calls at once and returns when the calls in flight have left.
    One condition variable guards everything; nothing is held while a backend releases its copies.
    """

    def __init__(self) -> None:
        self._cv = threading.Condition()
        self._entries: dict[int, _Entry] = {}
        self._handles = itertools.count(1)
        self._thread = threading.local()
        self._backends: dict[str, Callable[..., Any]] = {}

    # -- this thread's lease depth per handle
    def _depths(self) -> dict[int, int]:
        try:
            return self._thread.depths
        except AttributeError:
            self._thread.depths = {}
            return self._thread.depths

    def add(self, reader: Any) -> int:
        if getattr(reader, "mapping_count", None) != 1:
            raise ContractError("custom operator requires exactly one ExpertPack mapping")
        with self._cv:
            handle = next(self._handles)
            self._entries[handle] = _Entry(reader)
        return handle

    def remove(self, handle: int) -> None:
        if self._depths().get(handle):
            raise ContractError("cannot unregister an ExpertPack from its active call")
        with self._cv:
            entry = self._entries.get(handle)
            if entry is None:
                return
            if entry.closing:                       # another thread is closing it: leave when it is gone
                self._cv.wait_for(lambda: handle not in self._entries)
                return
            entry.closing = True
            self._cv.wait_for(lambda: entry.in_flight == 0)
            del self._entries[handle]
            listeners = [b for b in self._backends.values() if callable(getattr(b, "release_pack", None))]
            self._cv.notify_all()
        for backend in listeners:
            backend.release_pack(handle)

    @contextmanager
    def lease(self, handle: int) -> Iterator[Any]:
        depths = self._depths()
        outermost = depths.get(handle, 0) == 0
        with self._cv:
            entry = self._entries.get(handle)
            if entry is None or (entry.closing and outermost):
                raise RuntimeError(f"unknown or closed ExpertPack handle {handle}")
            if outermost:
                entry.in_flight += 1
        depths[handle] = depths.get(handle, 0) + 1
        try:
            yield entry.reader
        finally:
            depths[handle] -= 1
            if depths[handle] == 0:
                del depths[handle]
                with self._cv:
                    entry.in_flight -= 1
                    self._cv.notify_all()

    def reader(self, handle: int) -> Any:
        if not self._depths().get(handle):
            raise RuntimeError("ExpertPack access requires an active operator lease")
        with self._cv:
            entry = self._entries.get(handle)
        if entry is None:
            raise RuntimeError(f"unknown or closed ExpertPack handle {handle}")
        return entry.reader

    def set_backend(self, platform: str, implementation: Callable[..., Any]) -> None:
        if platform not in _KNOWN_PLATFORMS:
            raise ContractError(f"unsupported custom operator platform {platform!r}")
        if not callable(implementation):
            raise ContractError("custom operator backend must be callable")
        with self._cv:
            self._backends[platform] = implementation

    def backend(self, platform: str) -> Any:
        with self._cv:
            return self._backends.get(platform)


_REGISTRY = PackRegistry()
_LIBRARIES: list[Any] = []
_REGISTERED = False
_REGISTER_LOCK = threading.Lock()


# The reference's public functions (src/uma_qmoe/custom_op.py:51-146), same names, arguments and errors.

def register_expert_pack(reader: Any) -> int:
    return _REGISTRY.add(reader)


def register_target_pack(reader: Any) -> int:
    """A TargetPack registers exactly like an ExpertPack (one mapping, one handle)."""
    return _REGISTRY.add(reader)


def unregister_expert_pack(handle: int) -> None:
    """Close a handle: new calls are refused at once, the call returns when the
    calls in flight have drained, then every backend drops its device copies."""
    _REGISTRY.remove(handle)


def register_performance_backend(platform: str, implementation: Callable[..., Any]) -> None:
    """Install an explicit backend for a platform; never used as an implicit fallback."""
    _REGISTRY.set_backend(platform, implementation)


def acquire_expert_pack(handle: int):
    """Context manager that holds one pack open across staging and asynchronous kernel submission."""
    return _REGISTRY.lease(handle)


def expert_pack_for_handle(handle: int) -> Any:
    return _REGISTRY.reader(handle)


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
    return _REGISTRY.backend(platform)


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
    with _REGISTER_LOCK:
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
