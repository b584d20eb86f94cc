"""ctypes binding of ``libumaq_b200.so`` (the C ABI in ``include/umaq_b200.h``).

There is no fallback: if the library is missing the import of any operator
fails with an instruction to build it.
"""

from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

LIBRARY = Path(__file__).resolve().parent / "libumaq_b200.so"

ERRORS = {0: "ok", -1: "bad argument", -2: "workspace", -3: "launch failed", -4: "device-side wait timed out",
          -5: "unsupported"}


class Layer(C.Structure):
    _fields_ = [("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p),
                ("gate_scales", C.c_void_p), ("up_scales", C.c_void_p), ("down_scales", C.c_void_p),
                ("encoding", C.c_int32), ("num_experts", C.c_int32), ("hidden", C.c_int32),
                ("intermediate", C.c_int32)]


class EpPeers(C.Structure):
    _fields_ = [("base", C.c_void_p * 8), ("ranks", C.c_int32), ("rank", C.c_int32)]


class SharedExpert(C.Structure):
    _fields_ = [("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p), ("gate_vec", C.c_void_p),
                ("intermediate", C.c_int32)]


# name -> (restype, argtypes); every symbol include/umaq_b200.h declares
class PackTensor(C.Structure):
    """``umaq_pack_tensor``: one tensor of a mapped pack file."""

    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("data_bytes", C.c_size_t), ("scales", C.c_void_p),
                ("scale_bytes", C.c_size_t), ("encoding", C.c_int32), ("rank", C.c_int32), ("shape", C.c_longlong * 4),
                ("layer", C.c_int32), ("expert", C.c_int32), ("projection", C.c_int32)]


SIGNATURES = {
    "umaq_build_info": (C.c_int, [C.c_char_p, C.c_int]),
    "umaq_last_error": (C.c_char_p, []),
    "umaq_sm_count": (C.c_int, []),
    "umaq_decode_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "umaq_moe_decode": (C.c_int, [C.POINTER(Layer), C.POINTER(SharedExpert), C.c_void_p, C.c_void_p, C.c_int,
                                  C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "umaq_decode_plan": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int]),
    "umaq_moe_decode_static": (C.c_int, [C.POINTER(Layer), C.POINTER(SharedExpert), C.c_void_p, C.c_void_p, C.c_int,
                                         C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "umaq_route_topk": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                  C.c_void_p, C.c_void_p, C.c_void_p]),
    "umaq_prefill_workspace_bytes": (C.c_size_t, [C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "umaq_moe_prefill": (C.c_int, [C.POINTER(Layer), C.POINTER(SharedExpert), C.c_void_p, C.c_void_p, C.c_int,
                                   C.c_void_p, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "umaq_route_sort": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                  C.c_void_p, C.c_longlong, C.c_void_p]),
    "umaq_gather_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_void_p,
                                   C.c_void_p]),
    "umaq_grouped_gemm": (C.c_int, [C.POINTER(Layer), C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p,
                                    C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "umaq_grouped_gemm_by_index": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_void_p,
                                             C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "umaq_ep_local_ids": (C.c_int, [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                    C.c_void_p]),
    "umaq_ep_pack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                               C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "umaq_ep_push": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                               C.c_int, C.POINTER(EpPeers), C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]),
    "umaq_ep_barrier": (C.c_int, [C.POINTER(EpPeers), C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
    "umaq_moe_prefill_to_peers": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_longlong,
                                            C.c_int, C.POINTER(EpPeers), C.c_size_t, C.c_int, C.c_int, C.c_void_p,
                                            C.c_size_t, C.c_void_p]),
    "umaq_ep_layer": (C.c_int, [C.POINTER(Layer), C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                C.c_int, C.POINTER(EpPeers), C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                C.c_void_p]),
    "umaq_combine_routes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                      C.c_void_p, C.c_void_p]),
    "umaq_quantize_groups": (C.c_int, [C.c_void_p, C.c_longlong, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "umaq_probe_stream": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p]),
    "umaq_pack_open": (C.c_int, [C.c_char_p, C.c_int, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "umaq_pack_close": (None, [C.c_void_p]),
    "umaq_pack_tensor_count": (C.c_longlong, [C.c_void_p]),
    "umaq_pack_header_json": (C.c_void_p, [C.c_void_p, C.POINTER(C.c_size_t)]),
    "umaq_pack_layer_encoding": (C.c_int, [C.c_void_p, C.c_int]),
    "umaq_pack_tensor_view": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(PackTensor)]),
    "umaq_pack_tensor_at": (C.c_int, [C.c_void_p, C.c_longlong, C.POINTER(PackTensor)]),
    "umaq_sha256": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "umaq_stage_layer_async": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(Layer), C.c_int, C.POINTER(C.c_void_p)]),
    "umaq_stage_wait": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_double)]),
}


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    if not LIBRARY.exists():
        raise RuntimeError(
            f"{LIBRARY} is missing: the sm_100a kernels are not built and there is no fallback path. "
            "Run `python -m uma_qmoe_b200.build`.")
    handle = C.CDLL(str(LIBRARY))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)          # AttributeError if the library is stale
        fn.restype = restype
        fn.argtypes = argtypes
    return handle


def check(code: int, what: str) -> None:
    if code != 0:
        message = lib().umaq_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed ({ERRORS.get(code, code)}): {message}")
