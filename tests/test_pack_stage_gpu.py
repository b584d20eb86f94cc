"""Staging a layer from a pack file with the native reader (worker thread, pinned chunks, cudaMemcpyAsync per piece):
the device bytes must equal what the Python reader's path stages, for every encoding, and the operator on the staged
layer must give the result of the layer the file was written from."""

import pytest
import torch

from tests.helpers import SEED, assert_parity
from uma_qmoe_b200 import synthetic as syn

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _write_layer_pack(tmp_path, encoding: str):
    """An OLMoE-shaped layer 0 (64 experts) packed on the device and written with this package's writer."""
    from uma_qmoe_b200.formats import PackedTensor
    from uma_qmoe_b200.pack_writer import write_target_pack
    from uma_qmoe_b200.packs import expert_tensor_name
    from uma_qmoe_b200.stack import random_layer
    shape = syn.OLMOE
    source = random_layer(shape, encoding, SEED, DEV)
    per_expert = lambda t: None if t is None else t.reshape(-1).view(torch.uint8).cpu().numpy().reshape(shape.experts, -1)
    host = {p: (per_expert(getattr(source, p)), per_expert(getattr(source, p + "_scales"))) for p in ("gate", "up", "down")}

    def tensors():
        for e in range(shape.experts):
            for p in ("gate", "up", "down"):
                dims = (shape.hidden, shape.intermediate) if p == "down" else (shape.intermediate, shape.hidden)
                scales = b"" if host[p][1] is None else host[p][1][e].tobytes()
                yield expert_tensor_name(0, e, p + "_proj"), PackedTensor(encoding, dims, host[p][0][e].tobytes(), scales)
    path = tmp_path / f"layer0_{encoding}.uqmotpk"
    write_target_pack(path, tensors(), model_id="allenai/OLMoE-1B-7B-0125", model_revision="0" * 40,
                      model_manifest_sha256="0" * 64, policy_id="one-layer", layer_encodings={i: encoding for i in range(16)},
                      policy_evidence_sha256="0" * 64)
    return path, source


@pytest.mark.parametrize("encoding", ["q4_group128", "q8_group128", "bf16_le"])
def test_native_staging_equals_python_staging_and_runs(tmp_path, encoding):
    from uma_qmoe_b200 import custom_op, native_backend
    from uma_qmoe_b200.pack_files import NativeTargetPackFile, TargetPackFile
    path, source = _write_layer_pack(tmp_path, encoding)
    backend = native_backend.install_mixed_target_backend()
    x = syn.activations(SEED + 5, 24).to(DEV)
    g = torch.Generator().manual_seed(5)
    idx = torch.stack([torch.randperm(64, generator=g)[:8] for _ in range(24)]).to(DEV)
    w = torch.full((24, 8), 0.125, device=DEV)
    results = {}
    for name, cls in (("python", TargetPackFile), ("native", NativeTargetPackFile)):
        with cls(path, expected_policy_id="one-layer") as reader:
            handle = custom_op.register_target_pack(reader)
            try:
                if name == "native":
                    backend.prefetch_layer(handle, 0, DEV)                # starts the worker thread and returns
                y = torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True)
                one = torch.ops.uma_qmoe.moe_forward(x[:1], idx[:1], w[:1], 0, handle, True)
                with custom_op.acquire_expert_pack(handle) as r:
                    layer = backend._device_layer(handle, 0, DEV, r, "olmoe")
                for got, want in zip(layer.tensors, source.tensors):
                    assert torch.equal(got.reshape(-1).view(torch.uint8), want.reshape(-1).view(torch.uint8)), name
                results[name] = (y.clone(), one.clone())
                assert backend.cache_summary()["device_storage_bytes"] >= source.device_storage_bytes
            finally:
                custom_op.unregister_expert_pack(handle)
    assert torch.equal(results["python"][0], results["native"][0]) and torch.equal(results["python"][1], results["native"][1])
    from uma_qmoe_b200 import ops
    ws = ops.prefill_workspace(source, 24, 8, None, DEV)
    assert torch.equal(results["native"][0], ops.moe_prefill(source, x, idx, w, ws))
    assert_parity(results["native"][1].cpu(), results["native"][0][:1].cpu(), max_abs=2e-2)
