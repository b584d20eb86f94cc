"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol the header
declares, the operator registry mirrors the reference's registry / lease / fail-closed behaviour
(``src/uma_qmoe/custom_op.py``), and the host codecs agree with the reference-made golden vectors."""

import re
from pathlib import Path

import numpy as np
import pytest
import torch

from uma_qmoe_b200 import _native, custom_op, formats
from uma_qmoe_b200.formats import ContractError

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols() -> list[str]:
    text = (ROOT / "include" / "umaq_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(umaq_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_without_a_gpu_and_exports_every_declared_symbol():
    lib = _native.lib()
    declared = _declared_symbols()
    assert len(declared) >= 14
    assert sorted(_native.SIGNATURES) == declared, "ctypes table and header must list the same entry points"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/umaq_b200.h but not exported"


def test_header_constants_match_the_python_side():
    """The flag and error values the Python wrappers pass are the ones the header defines."""
    from uma_qmoe_b200 import ops
    text = (ROOT / "include" / "umaq_b200.h").read_text()
    defines = {name: int(value) for name, value in re.findall(r"^#define\s+(UMAQ_[A-Z0-9_]+)\s+(-?\d+)\s*$", text, flags=re.M)}
    assert defines["UMAQ_EP_LOCAL_IDS"] == ops.EP_LOCAL_IDS
    assert defines["UMAQ_EP_K_PERMUTED"] == ops.EP_K_PERMUTED
    assert ops.EP_LOCAL_IDS & ops.EP_K_PERMUTED == 0


def test_build_info_names_the_target_and_the_source_digest():
    from uma_qmoe_b200 import build
    lib = _native.lib()
    import ctypes as C
    raw = C.create_string_buffer(512)
    n = lib.umaq_build_info(raw, 512)
    info = raw.value.decode()
    assert n > 0 and "sm_100a" in info
    assert len(build.source_sha256()) == 64


def test_workspace_sizes_are_host_arithmetic():
    lib = _native.lib()
    # header + four bytes per intermediate value (slot count rounded up to a power of two) + alignment slack
    assert lib.umaq_decode_workspace_bytes(8, 1024, 0) == 1024 + 8 * 1024 * 4 + 512
    assert lib.umaq_decode_workspace_bytes(4, 1408, 5632) == 1024 + (4 * 1408 + 5632) * 4 + 512
    assert lib.umaq_decode_workspace_bytes(6, 1024, 0) == 1024 + 8 * 1024 * 4 + 512
    assert lib.umaq_decode_workspace_bytes(4, 1408, 5632) <= 64 * 1024        # fits the built-in scratch block
    small = lib.umaq_prefill_workspace_bytes(1, 8, 64, 2048, 1024, 0)
    big = lib.umaq_prefill_workspace_bytes(8192, 8, 64, 2048, 1024, 0)
    assert 0 < small < big
    # sorted activations + intermediate + weighted outputs dominate: routes * (H + I + H) * 2 bytes
    assert big >= 65536 * (2048 + 1024 + 2048) * 2


def test_decode_launch_plans_fit_one_sm_together():
    """Host arithmetic of the decode launcher: for every shape of the benchmark configurations the two kernels'
    shared memory fits one SM side by side, every CTA's share fits its ring or the ring has at least two stages,
    and the work is spread over all SMs."""
    import ctypes as C
    lib = _native.lib()
    out = (C.c_int * 12)()
    shapes = {"olmoe q4": (0, 2048, 1024, 8, 0), "olmoe q8": (1, 2048, 1024, 8, 0), "olmoe bf16": (2, 2048, 1024, 8, 0),
              "qwen q8 + shared": (1, 2048, 1408, 4, 5632), "qwen bf16 + shared": (2, 2048, 1408, 4, 5632),
              "qwen q4 + shared": (0, 2048, 1408, 4, 5632), "small": (0, 512, 256, 2, 0)}
    for name, args in shapes.items():
        assert lib.umaq_decode_plan(*args, 148, out, 12) == 0, (name, lib.umaq_last_error())
        g_grid, g_stages, g_stage, g_smem, g_units, g_ips, d_grid, d_stages, d_stage, d_smem, d_units, d_ips = list(out)
        assert g_smem + d_smem <= 226 * 1024, name
        # the down kernel reports one "stage" when it holds a CTA's whole share at once (no ring)
        assert g_stages >= min(2, g_units) and (d_stages >= min(2, d_units) or d_stages == 1), name
        # one gate/up CTA per SM; the down kernel takes two per SM when there is a shared expert (ring mode)
        assert 1 <= g_grid <= 148 and 1 <= d_grid <= (296 if args[4] else 148), name
    assert lib.umaq_decode_plan(0, 2048, 1024, 8, 0, 148, out, 12) == 0
    assert list(out)[:2] == [148, 7] and list(out)[6:8] == [148, 1]        # OLMoE: a CTA's whole share is in flight at once
    assert lib.umaq_decode_plan(0, 2048, 1000, 8, 0, 148, out, 12) == -1   # intermediate not a multiple of 128
    assert lib.umaq_decode_plan(0, 2048, 1024, 9, 0, 148, out, 12) == -1   # more than 8 routes


class _Reader:
    mapping_count = 1


def test_registry_handles_leases_and_unregister():
    with pytest.raises(ContractError, match="exactly one ExpertPack mapping"):
        custom_op.register_expert_pack(object())
    handle = custom_op.register_expert_pack(_Reader())
    other = custom_op.register_target_pack(_Reader())
    assert other != handle
    with pytest.raises(RuntimeError, match="active operator lease"):
        custom_op.expert_pack_for_handle(handle)
    with custom_op.acquire_expert_pack(handle) as reader:
        assert isinstance(reader, _Reader)
        assert custom_op.expert_pack_for_handle(handle) is reader
        with pytest.raises(ContractError, match="active call"):
            custom_op.unregister_expert_pack(handle)
    custom_op.unregister_expert_pack(handle)
    custom_op.unregister_expert_pack(other)
    with pytest.raises(RuntimeError, match="unknown or closed ExpertPack handle"):
        with custom_op.acquire_expert_pack(handle):
            pass


def test_backend_registration_checks_platform_and_callable():
    with pytest.raises(ContractError, match="unsupported custom operator platform"):
        custom_op.register_performance_backend("tpu_v5", lambda *a: None)
    with pytest.raises(ContractError, match="must be callable"):
        custom_op.register_performance_backend("cuda_sm100", 3)


def test_operators_fail_closed_on_cpu_tensors():
    """No backend is registered for CPU tensors and there is no reference fallback in this package:
    both operators must raise the reference's fail-closed message instead of computing anything."""
    custom_op.register_moe_forward()
    handle = custom_op.register_expert_pack(_Reader())
    try:
        x = torch.zeros((1, 2048), dtype=torch.bfloat16)
        idx = torch.zeros((1, 8), dtype=torch.int64)
        w = torch.zeros((1, 8), dtype=torch.float32)
        with pytest.raises(RuntimeError, match="performance mode has no registered cpu backend; "
                                               "silent reference fallback is forbidden"):
            torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True)
        with pytest.raises(RuntimeError, match="silent reference fallback is forbidden"):
            torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, False)
        with pytest.raises(RuntimeError, match="performance mode has no Qwen-capable cpu backend"):
            torch.ops.uma_qmoe.qwen_moe_forward(x, idx, w, 0, handle, True)
    finally:
        custom_op.unregister_expert_pack(handle)


def test_operator_schemas_match_the_reference():
    custom_op.register_moe_forward()
    want = ("(Tensor hidden_states, Tensor expert_indices, Tensor routing_weights, int layer_index, "
            "int pack_handle, bool performance_mode=False) -> Tensor")
    for op in (torch.ops.uma_qmoe.moe_forward, torch.ops.uma_qmoe.qwen_moe_forward):
        assert str(op.default._schema).endswith(want)


def test_product_package_never_imports_the_oracle():
    for path in (ROOT / "uma_qmoe_b200").rglob("*.py"):
        text = path.read_text()
        assert "oracle" not in re.sub(r"#.*", "", text), f"{path} refers to the test oracle"


def test_host_codecs_reproduce_the_golden_bytes(golden_dir):
    """``formats.encode`` (what the native backend's staging and the synthetic packs use) against the
    reference's own encoders on the four golden inputs (1, 129, 255 and 1000 values)."""
    g = np.load(golden_dir / "codec.npz")
    for i in range(4):
        v = g[f"in_{i}"]
        q4 = formats.encode(v, "q4_group128")
        assert bytes(q4.data) == g[f"q4_packed_{i}"].tobytes()
        assert np.array_equal(np.frombuffer(q4.scales, np.float32), g[f"q4_scales_{i}"])
        q8 = formats.encode(v, "q8_group128")
        assert bytes(q8.data) == g[f"q8_data_{i}"].tobytes()
        assert np.array_equal(np.frombuffer(q8.scales, np.float32), g[f"q8_scales_{i}"])
        bf = formats.encode(v, "bf16_le")
        assert bytes(bf.data) == g[f"bf16_{i}"].astype("<u2").tobytes()
        for packed in (q4, q8, bf):
            back = formats.decode(packed)
            assert back.shape == v.shape and np.isfinite(back).all()
            bound = np.abs(v).max() / (7 if packed is q4 else 127) if packed is not bf else np.abs(v).max() * 2 ** -8
            assert np.abs(back - v).max() <= bound + 1e-12


def test_unregister_waits_for_the_call_in_flight_and_refuses_new_calls():
    """``src/uma_qmoe`` lifecycle contract (the reference's ``test_custom_operator_lifecycle.py:37-67``): closing a
    handle blocks until the active call has left, and nobody can enter in between."""
    import threading
    handle = custom_op.register_expert_pack(_Reader())
    entered, release, closed = threading.Event(), threading.Event(), threading.Event()

    def call():
        with custom_op.acquire_expert_pack(handle):
            entered.set()
            assert release.wait(timeout=5)

    def close():
        custom_op.unregister_expert_pack(handle)
        closed.set()

    worker, closer = threading.Thread(target=call), threading.Thread(target=close)
    worker.start()
    assert entered.wait(timeout=5)
    closer.start()
    assert not closed.wait(timeout=0.1)
    with pytest.raises(RuntimeError, match="unknown or closed"):
        with custom_op.acquire_expert_pack(handle):
            pass
    release.set()
    worker.join(timeout=5)
    closer.join(timeout=5)
    assert not worker.is_alive() and not closer.is_alive() and closed.is_set()


def test_backend_needs_every_entry_point_and_drops_the_caches_of_a_closed_pack():
    from types import SimpleNamespace
    from uma_qmoe_b200.native_backend import MixedTargetNativeBackend, PackedQ4NativeBackend
    with pytest.raises(ContractError, match="unsupported native platform"):
        MixedTargetNativeBackend("cuda_sm121", _native.lib())
    partial = SimpleNamespace(**{name: None for name in list(_native.SIGNATURES)[:-1]})
    with pytest.raises(ContractError, match="does not export"):
        MixedTargetNativeBackend("cuda_sm100", partial)
    backend = PackedQ4NativeBackend("cuda_sm100", _native.lib())
    assert backend.allowed_encodings == ("q4_group128",)
    layer = SimpleNamespace(num_experts=64, device_storage_bytes=10)
    backend.preload_layer(1, 0, "cuda:0", layer)
    backend.preload_layer(1, 5, "cuda:0", layer)
    backend.preload_layer(2, 0, "cuda:0", layer)
    assert backend.cache_summary() == {"tensor_count": 3 * 64 * 3, "device_storage_bytes": 30, "dequantized_weight_bytes": 0}
    backend.release_pack(1)
    assert backend.cache_summary()["device_storage_bytes"] == 10
