"""Batch-1 decode kernel vs the CPU oracle and the reference-made golden vectors (through the C ABI)."""

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.helpers import SEED, assert_parity, bits_to_bf16, expert_source, stage_layer
from uma_qmoe_b200 import synthetic as syn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ops():
    from uma_qmoe_b200 import ops
    return ops


def _run_decode(layer, x, idx, w, shared=None):
    ops = _ops()
    ws = ops.decode_workspace(layer, idx.numel(), shared, torch.device(DEV))
    y = ops.moe_decode(layer, x.to(DEV).contiguous(), idx.to(DEV).contiguous(), w.to(DEV).contiguous(), ws, shared)
    y2 = ops.moe_decode(layer, x.to(DEV).contiguous(), idx.to(DEV).contiguous(), w.to(DEV).contiguous(), ws, shared)
    torch.cuda.synchronize()
    assert ops.workspace_status(ws) == 0
    assert torch.equal(y, y2), "two calls on one workspace must give identical bits"
    return y.cpu()


def test_device_packer_bit_exact():
    ops = _ops()
    v = torch.from_numpy(syn.normal_bf16((SEED, 77), (64, 1024), 0.02))
    v[3, :128] = 0.0
    v[5, 128:256] = 1e-30
    vb = v.to(torch.bfloat16)
    for enc, ref in (("q4_group128", orc.quantize_q4), ("q8_group128", orc.quantize_q8)):
        codes, scales = ops.quantize_groups(vb.to(DEV), enc)
        want_codes, want_scales = ref(vb.float().numpy())
        assert np.array_equal(codes.cpu().numpy().view(np.uint8), np.asarray(want_codes).view(np.uint8)), enc
        assert np.array_equal(scales.cpu().numpy(), want_scales), enc


def test_olmoe_decode_golden(golden_dir):
    g = np.load(golden_dir / "olmoe_decode.npz")
    x = bits_to_bf16(g["x_bits"])
    idx = torch.from_numpy(g["idx"])
    src = expert_source(SEED, 0, "olmoe", "q4_group128")
    experts = {int(e): src(int(e)) for e in set(idx.reshape(-1).tolist())}
    layer = stage_layer(experts, 64, 2048, 1024, "q4_group128", DEV)
    for wkey, ykey in (("w_norm", "y_norm_bits"), ("w_raw", "y_raw_bits")):
        y = _run_decode(layer, x, idx, torch.from_numpy(g[wkey]))
        m = assert_parity(y, bits_to_bf16(g[ykey]))
        assert m["max_abs"] <= 4e-3, m          # the kernel keeps the oracle's rounding points


def test_olmoe_decode_int32_duplicate_and_order():
    src = expert_source(SEED, 5, "olmoe", "q4_group128")
    idx = torch.tensor([[9, 2, 2, 7, 0, 11, 4, 1]], dtype=torch.int32)
    w = torch.tensor([[0.3, 0.05, 0.1, 0.2, 0.05, 0.1, 0.15, 0.05]])
    experts = {int(e): src(int(e)) for e in set(idx.reshape(-1).tolist())}
    layer = stage_layer(experts, 16, 2048, 1024, "q4_group128", DEV)
    x = syn.activations(SEED + 11, 1)
    want = orc.moe_forward(x, idx.long(), w, src, num_experts=64, top_k=8, qwen=False)
    assert_parity(_run_decode(layer, x, idx, w), want)


@pytest.mark.parametrize("encoding", ["q8_group128", "bf16_le"])
def test_olmoe_shape_other_encodings(encoding):
    src = expert_source(SEED, 6, "olmoe", encoding)
    idx = torch.tensor([[3, 1, 0, 2, 5, 4, 7, 6]])
    w = torch.full((1, 8), 0.125)
    layer = stage_layer({e: src(e) for e in range(8)}, 8, 2048, 1024, encoding, DEV)
    x = syn.activations(SEED + 12, 1)
    want = orc.moe_forward(x, idx, w, src, num_experts=64, top_k=8, qwen=False)
    assert_parity(_run_decode(layer, x, idx, w), want)


def test_large_activations_do_not_overflow():
    src = expert_source(SEED, 6, "olmoe", "q4_group128")
    idx = torch.tensor([[3, 1, 0, 2, 5, 4, 7, 6]])
    w = torch.full((1, 8), 0.125)
    layer = stage_layer({e: src(e) for e in range(8)}, 8, 2048, 1024, "q4_group128", DEV)
    x = (syn.activations(SEED + 13, 1).float() * 3000.0).to(torch.bfloat16)
    want = orc.moe_forward(x, idx, w, src, num_experts=64, top_k=8, qwen=False)
    got = _run_decode(layer, x, idx, w)
    m = orc.compare(got, want)
    assert m["cosine"] >= 0.9999 and torch.isfinite(got.float()).all(), m


@pytest.mark.parametrize("layer_index", [0, 1, 2])
def test_qwen_decode_golden(golden_dir, layer_index):
    from uma_qmoe_b200.ops import DeviceSharedExpert
    g = np.load(golden_dir / "qwen_layers.npz")
    enc = str(g[f"L{layer_index}_encoding"])
    src = expert_source(SEED, layer_index, "qwen", enc)
    x = bits_to_bf16(g["x1_bits"])
    idx = torch.from_numpy(g[f"L{layer_index}_i1"])
    w = torch.from_numpy(g[f"L{layer_index}_w1"])
    experts = {int(e): src(int(e)) for e in set(idx.reshape(-1).tolist())}
    layer = stage_layer(experts, 60, 2048, 1408, enc, DEV)
    y = _run_decode(layer, x, idx, w)
    assert_parity(y, bits_to_bf16(g[f"L{layer_index}_y1_bits"]))
    sg, su, sd, sgate = (t.to(DEV).contiguous() for t in syn.shared_expert_weights(SEED, layer_index, syn.QWEN))
    shared = DeviceSharedExpert(sg, su, sd, sgate)
    b = _run_decode(layer, x, idx, w, shared)
    assert_parity(b, bits_to_bf16(g[f"L{layer_index}_b1_bits"]))


def test_bad_expert_index_sets_status_and_does_not_hang():
    ops = _ops()
    src = expert_source(SEED, 6, "olmoe", "q4_group128")
    layer = stage_layer({0: src(0)}, 4, 2048, 1024, "q4_group128", DEV)
    ws = ops.decode_workspace(layer, 8, None, torch.device(DEV))
    idx = torch.tensor([[0, 1, 2, 3, 0, 1, 2, 99]], device=DEV)
    ops.moe_decode(layer, syn.activations(1, 1).to(DEV), idx, torch.full((1, 8), 0.125, device=DEV), ws)
    torch.cuda.synchronize()
    assert ops.workspace_status(ws) == -1


def test_rejects_cpu_tensors_and_bad_shapes():
    ops = _ops()
    src = expert_source(SEED, 6, "olmoe", "q4_group128")
    layer = stage_layer({0: src(0)}, 1, 2048, 1024, "q4_group128", DEV)
    ws = ops.decode_workspace(layer, 8, None, torch.device(DEV))
    idx = torch.zeros((1, 8), dtype=torch.int64, device=DEV)
    w = torch.full((1, 8), 0.125, device=DEV)
    with pytest.raises(RuntimeError):
        ops.moe_decode(layer, syn.activations(1, 1), idx, w, ws)               # CPU tensor: no fallback
    with pytest.raises(RuntimeError):
        ops.moe_decode(layer, syn.activations(1, 2).to(DEV), idx, w, ws)       # two tokens
    with pytest.raises(RuntimeError):
        ops.moe_decode(layer, syn.activations(1, 1).to(DEV), idx, w, ws[:64])  # workspace too small


def test_reference_validator_and_route_trace_decode(golden_dir):
    """One token of the reference validator's inputs (linspace hidden state, experts 0..7, weights 0.125) and the
    first decode event of layer 0 of the reference's frozen route trace, against the reference's CPU outputs."""
    g = np.load(golden_dir / "reference_cases.npz")
    src = expert_source(SEED, int(g["layer"]), "olmoe", "q4_group128")
    layer = stage_layer({int(e): src(int(e)) for e in g["hit"]}, 64, 2048, 1024, "q4_group128", DEV)
    y = _run_decode(layer, bits_to_bf16(g["val_x1_bits"]), torch.from_numpy(g["val_idx"]),
                    bits_to_bf16(g["val_w_bits"]).float())
    assert_parity(y, bits_to_bf16(g["val_y1_bits"]))
    y = _run_decode(layer, bits_to_bf16(g["trace_decode_x_bits"]), torch.from_numpy(g["trace_decode_idx"]),
                    torch.from_numpy(g["trace_decode_w"]))
    assert_parity(y, bits_to_bf16(g["trace_decode_y_bits"]))


def test_bad_expert_index_is_skipped_like_the_reference():
    """An out-of-range index contributes nothing (the reference's kernels skip it,
    src/uma_qmoe/native/packed_q4_kernel.cu:176); the other routes still produce the complete output."""
    ops = _ops()
    src = expert_source(SEED, 6, "olmoe", "q4_group128")
    layer = stage_layer({e: src(e) for e in range(4)}, 4, 2048, 1024, "q4_group128", DEV)
    x = syn.activations(SEED + 14, 1)
    idx = torch.tensor([[0, 1, 2, 3, 0, 1, 2, 99]])
    w = torch.full((1, 8), 0.125)
    ws = ops.decode_workspace(layer, 8, None, torch.device(DEV))
    y = ops.moe_decode(layer, x.to(DEV), idx.to(DEV), w.to(DEV), ws).cpu()
    torch.cuda.synchronize()
    assert ops.workspace_status(ws) == -1
    want = orc.moe_forward(x, idx[:, :7].contiguous(), w[:, :7].contiguous(), src, num_experts=64, top_k=7, qwen=False)
    assert_parity(y, want)
