"""Pin the CPU oracle: its codecs, router and operator restatements must
reproduce what the reference itself produced for the golden fixtures, and the
reference's own known-answer vectors."""

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.helpers import SEED, bf16_bits, bits_to_bf16, expert_source, sha, ulp_bf16
from uma_qmoe_b200 import synthetic as syn


# ---- known-answer vectors of the reference's own unit tests -------------------

def test_q4_nibble_order_known_answer():
    # reference tests/unit/test_q4.py:19-23
    assert bytes(orc.pack_int4(np.array([-7, -1, 0, 1, 7]))) == bytes([0xF9, 0x10, 0x07])
    assert orc.unpack_int4(np.array([0xF9, 0x10, 0x07], np.uint8), 5).tolist() == [-7, -1, 0, 1, 7]


def test_q4_tail_group_and_error_bound():
    # reference tests/unit/test_q4.py:26-40: 129 elements -> 65 packed bytes, 2 scales
    v = np.linspace(-1, 1, 129, dtype=np.float32)
    packed, scales = orc.quantize_q4(v)
    assert packed.size == 65 and scales.size == 2
    back = orc.dequantize_q4(packed, scales, (129,))
    assert np.all(np.abs(back - v) <= np.repeat(scales, 128)[:129] / 2 + 1e-7)


def test_q4_reserved_code_and_tail_padding_rejected():
    # reference tests/unit/test_q4.py:43-47
    with pytest.raises(ValueError):
        orc.unpack_int4(np.array([0x08], np.uint8), 2)
    with pytest.raises(ValueError):
        orc.unpack_int4(np.array([0x10], np.uint8), 1)


def test_q4_zero_group_scale_is_one():
    # reference tests/unit/test_q4.py:50-55
    packed, scales = orc.quantize_q4(np.zeros(128, np.float32))
    assert scales.tolist() == [1.0] and not packed.any()
    assert not orc.dequantize_q4(packed, scales, (128,)).any()


def test_q8_known_answer():
    # reference tests/unit/test_target_pack.py:140-166: bytes (1, 255), scale 0.25 -> (0.25, -0.25)
    out = orc.dequantize_q8(np.array([1, 255], np.uint8), np.array([0.25], "<f4"), (2,))
    assert out.tolist() == [0.25, -0.25]


def test_bf16_error_bound():
    # reference tests/unit/test_target_pack.py:83-86
    v = np.linspace(-1, 1, 257, dtype=np.float32)
    back = orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(v), v.shape)
    assert np.abs(back - v).max() < 0.01


# ---- golden vectors produced by the reference ---------------------------------

def test_codecs_bit_exact(golden_dir):
    g = np.load(golden_dir / "codec.npz")
    for i in range(4):
        v = g[f"in_{i}"]
        packed, scales = orc.quantize_q4(v)
        assert np.array_equal(packed, g[f"q4_packed_{i}"]) and np.array_equal(scales, g[f"q4_scales_{i}"])
        codes, s8 = orc.quantize_q8(v)
        assert np.array_equal(codes, g[f"q8_data_{i}"]) and np.array_equal(s8, g[f"q8_scales_{i}"])
        assert np.array_equal(orc.f32_to_bf16_bits(v), g[f"bf16_{i}"])


def _assert_close_bf16(actual: torch.Tensor, expected: torch.Tensor, ulps: int = 2):
    """Bit-exact on the torch build that made the fixtures; a different CPU
    GEMM kernel may move a result by an ulp, never more."""
    diff = (actual.float() - expected.float()).abs()
    assert bool((diff <= ulps * ulp_bf16(expected)).all()), float(diff.max())


def test_olmoe_decode_matches_reference(golden_dir):
    g = np.load(golden_dir / "olmoe_decode.npz")
    x = bits_to_bf16(g["x_bits"])
    wr = syn.router_weight(SEED, 0, syn.OLMOE)
    assert sha(bf16_bits(wr).tobytes()) == str(g["router_sha"])
    probs, w, idx = orc.router_topk(x, wr, 8, True)
    assert np.array_equal(idx.numpy(), g["idx"])
    assert np.array_equal(w.numpy(), g["w_norm"])
    _p, w_raw, idx_raw = orc.router_topk(x, wr, 8, False)
    assert np.array_equal(idx_raw.numpy(), g["idx"]) and np.array_equal(w_raw.numpy(), g["w_raw"])
    src = expert_source(SEED, 0, "olmoe", "q4_group128")
    for e in sorted(set(g["idx"].reshape(-1).tolist())):
        for m, p in zip(src(e), ("gate", "up", "down")):
            assert sha(m.data.tobytes(), m.scales.tobytes()) == str(g[f"sha_{e}_{p}"])
    y = orc.moe_forward(x, idx, w, src, num_experts=64, top_k=8, qwen=False)
    _assert_close_bf16(y, bits_to_bf16(g["y_norm_bits"]))
    y = orc.moe_forward(x, idx, w_raw, src, num_experts=64, top_k=8, qwen=False)
    _assert_close_bf16(y, bits_to_bf16(g["y_raw_bits"]))


def test_olmoe_prefill_matches_reference(golden_dir):
    g = np.load(golden_dir / "olmoe_prefill.npz")
    x = bits_to_bf16(g["x_bits"])
    idx, w = torch.from_numpy(g["idx"]), torch.from_numpy(g["w"])
    src = expert_source(SEED, 3, "olmoe", "q4_group128")
    y = orc.moe_forward(x, idx, w, src, num_experts=64, top_k=8, qwen=False)
    _assert_close_bf16(y, bits_to_bf16(g["y_bits"]))
    counts = torch.bincount(idx.reshape(-1), minlength=64)
    assert int((counts == 0).sum()) >= 52 and int(counts.max()) >= 3 * counts.float().mean()


@pytest.mark.parametrize("layer", [0, 1, 2])
def test_qwen_layers_match_reference(golden_dir, layer):
    g = np.load(golden_dir / "qwen_layers.npz")
    enc = str(g[f"L{layer}_encoding"])
    src = expert_source(SEED, layer, "qwen", enc)
    wr = syn.router_weight(SEED, layer, syn.QWEN)
    sg, su, sd, sgate = syn.shared_expert_weights(SEED, layer, syn.QWEN)
    for tag in ("1", "8"):
        x = bits_to_bf16(g[f"x{tag}_bits"])
        _p, w, idx = orc.router_topk(x, wr, 4, False)
        assert np.array_equal(idx.numpy(), g[f"L{layer}_i{tag}"])
        assert np.array_equal(w.numpy(), g[f"L{layer}_w{tag}"])
        y = orc.moe_forward(x, idx, w, src, num_experts=60, top_k=4, qwen=True)
        _assert_close_bf16(y, bits_to_bf16(g[f"L{layer}_y{tag}_bits"]))
        b = orc.qwen_block_forward(x, wr, sg, su, sd, sgate, src)
        _assert_close_bf16(b, bits_to_bf16(g[f"L{layer}_b{tag}_bits"]))
    for e in sorted(set(g[f"L{layer}_i1"].reshape(-1).tolist())):
        for m, p in zip(src(e), ("gate", "up", "down")):
            assert sha(m.data.tobytes(), m.scales.tobytes()) == str(g[f"L{layer}_sha_{e}_{p}"])


def test_sorted_routes_is_stable_counting_sort():
    idx = torch.tensor([[3, 1], [1, 0], [3, 3]])
    order, offsets = orc.sorted_routes(idx, 4)
    assert order.tolist() == [3, 1, 2, 0, 4, 5]
    assert offsets.tolist() == [0, 1, 3, 3, 6]


def test_reference_validator_and_route_trace_cases(golden_dir):
    """The reference validator's own inputs (benchmarks/runners/validate_packed_q4_kernel.py:151-178) and one
    layer of its frozen route trace (src/uma_qmoe/route_trace.py:382-404), outputs made by the reference."""
    g = np.load(golden_dir / "reference_cases.npz")
    src = expert_source(SEED, int(g["layer"]), "olmoe", "q4_group128")
    idx = torch.from_numpy(g["val_idx"])
    w = bits_to_bf16(g["val_w_bits"])                       # the validator passes BF16 routing weights
    y = orc.moe_forward(bits_to_bf16(g["val_x1_bits"]), idx, w, src, num_experts=64, top_k=8, qwen=False)
    _assert_close_bf16(y, bits_to_bf16(g["val_y1_bits"]))
    y = orc.moe_forward(bits_to_bf16(g["val_x32_bits"]), idx.repeat(32, 1), w.repeat(32, 1), src, num_experts=64,
                        top_k=8, qwen=False)
    _assert_close_bf16(y, bits_to_bf16(g["val_y32_bits"]))
    for phase in ("prefill", "decode"):
        idx = torch.from_numpy(g[f"trace_{phase}_idx"])
        w = torch.from_numpy(g[f"trace_{phase}_w"])
        y = orc.moe_forward(bits_to_bf16(g[f"trace_{phase}_x_bits"]), idx, w, src, num_experts=64, top_k=8, qwen=False)
        _assert_close_bf16(y, bits_to_bf16(g[f"trace_{phase}_y_bits"]))
    counts = torch.bincount(torch.from_numpy(g["trace_prefill_idx"]).reshape(-1), minlength=64)
    assert int((counts > 0).sum()) == 32 and int(counts.max()) == 53      # the skew the survey quotes for this layer
    assert abs(float(g["trace_prefill_w"][0].sum()) - 1.0) > 0.1          # real routes are not renormalised
