"""The decode entry point that brings its own scratch (``umaq_moe_decode_static``).

Some hosts of this library may not allocate device memory at the point where they call it -- a
plug-in running inside another runtime's stream hook only gets its input and output buffers.  For
them the library carries a fixed 64 KiB scratch block per device.  This test calls that entry point
through the C ABI twice in a row and compares each result with the regular entry point (which works
in a caller-provided workspace); both run the same kernel, so the outputs must agree bit for bit,
and they must also meet the operator's tolerance against the CPU oracle.  The file sorts last so a
run that stops at the first failure has already covered everything else.
"""

import ctypes as C

import pytest
import torch

from oracle import moe_oracle as orc
from tests.helpers import SEED, assert_parity, expert_source, stage_layer
from uma_qmoe_b200 import synthetic as syn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call_static(layer, x, idx, w, shared=None):
    from uma_qmoe_b200 import _native
    out = torch.empty_like(x)
    stream = C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    code = _native.lib().umaq_moe_decode_static(C.byref(layer.struct()),
                                                C.byref(shared.struct()) if shared is not None else None,
                                                x.data_ptr(), idx.data_ptr(),
                                                int(idx.dtype == torch.int64), w.data_ptr(), idx.numel(),
                                                out.data_ptr(), stream)
    _native.check(code, "umaq_moe_decode_static")
    return out


def test_static_scratch_decode_matches_workspace_decode_twice():
    from uma_qmoe_b200 import ops
    src = expert_source(SEED, 6, "olmoe", "q4_group128")
    layer = stage_layer({e: src(e) for e in range(8)}, 8, 2048, 1024, "q4_group128", DEV)
    ws = ops.decode_workspace(layer, 8, None, torch.device(DEV))
    for call in range(2):                       # second call starts from the first call's leftovers
        x = syn.activations(SEED + 40 + call, 1)
        idx = torch.tensor([[3, 1, 0, 2, 5, 4, 7, 6]]).roll(call, dims=1).contiguous()
        w = torch.full((1, 8), 0.125) + 0.01 * call
        xd, idd, wd = x.to(DEV), idx.to(DEV), w.to(DEV)
        got = _call_static(layer, xd, idd, wd)
        ref = ops.moe_decode(layer, xd, idd, wd, ws)
        torch.cuda.synchronize()
        assert torch.equal(got, ref), f"call {call}: static-scratch result differs from the workspace result"
        assert_parity(got.cpu(), orc.moe_forward(x, idx, w, src, num_experts=64, top_k=8, qwen=False))


def test_static_scratch_decode_with_the_qwen_shared_expert():
    """The largest shape the header names for this entry point: four Q8 experts of 1408 plus the BF16 shared
    expert of 5632 with its sigmoid gate.  Two calls in a row, each bit-equal to the workspace entry point."""
    from uma_qmoe_b200 import ops
    from uma_qmoe_b200.ops import DeviceSharedExpert
    src = expert_source(SEED, 1, "qwen", "q8_group128")
    layer = stage_layer({e: src(e) for e in range(6)}, 6, 2048, 1408, "q8_group128", DEV)
    sg, su, sd, sgate = (t.to(DEV).contiguous() for t in syn.shared_expert_weights(SEED, 1, syn.QWEN))
    shared = DeviceSharedExpert(sg, su, sd, sgate)
    ws = ops.decode_workspace(layer, 4, shared, torch.device(DEV))
    for call in range(2):
        x = syn.activations(SEED + 50 + call, 1)
        idx = torch.tensor([[5, 0, 3, 2]]).roll(call, dims=1).contiguous()
        w = torch.tensor([[0.4, 0.3, 0.2, 0.1]]) + 0.01 * call
        xd, idd, wd = x.to(DEV), idx.to(DEV), w.to(DEV)
        got = _call_static(layer, xd, idd, wd, shared)
        ref = ops.moe_decode(layer, xd, idd, wd, ws, shared)
        torch.cuda.synchronize()
        assert torch.equal(got, ref), f"call {call}: static-scratch result differs from the workspace result"
        # routed experts plus the shared branch of QuantizedQwenMoEBlock (BF16 linears, sigmoid gate), on the CPU
        F = torch.nn.functional
        hg, hu, hd, hgate = syn.shared_expert_weights(SEED, 1, syn.QWEN)
        want = orc.moe_forward(x, idx, w, src, num_experts=60, top_k=4, qwen=True)
        want = want + torch.sigmoid(F.linear(x, hgate)) * F.linear(F.silu(F.linear(x, hg)) * F.linear(x, hu), hd)
        assert_parity(got.cpu(), want)


def test_static_scratch_rejects_shapes_beyond_its_block():
    from uma_qmoe_b200 import _native
    src = expert_source(SEED, 6, "olmoe", "q4_group128")
    layer = stage_layer({0: src(0)}, 1, 2048, 1024, "q4_group128", DEV)
    big = layer.struct()
    big.intermediate = 4096                      # 8 x 4096 float32 values do not fit 64 KiB
    x = syn.activations(1, 1).to(DEV)
    idx = torch.zeros((1, 8), dtype=torch.int64, device=DEV)
    w = torch.full((1, 8), 0.125, device=DEV)
    out = torch.empty_like(x)
    code = _native.lib().umaq_moe_decode_static(C.byref(big), None, x.data_ptr(), idx.data_ptr(), 1, w.data_ptr(), 8,
                                                out.data_ptr(), None)
    assert code == -2
    assert b"64" in _native.lib().umaq_last_error() or b"65536" in _native.lib().umaq_last_error()
