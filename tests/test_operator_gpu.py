"""The registered operator under the conditions a serving host puts it in: calls from several threads on several
streams at once, device-side errors reported without a wait on the hot path, BF16 routing weights."""

import threading

import pytest
import torch

from tests.helpers import SEED, assert_parity
from uma_qmoe_b200 import synthetic as syn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def olmoe_pack():
    """A one-layer Q4 pack (8 distinct experts repeated to fill the layer's 64) behind the installed back end."""
    from uma_qmoe_b200 import custom_op, native_backend
    from uma_qmoe_b200.formats import encode
    from uma_qmoe_b200.packs import InMemoryPack, expert_tensor_name
    pack = InMemoryPack({0: "q4_group128"})
    packed = {}
    for e in range(8):
        for proj, m in zip(("gate_proj", "up_proj", "down_proj"), syn.expert_weights(SEED, 0, e, syn.OLMOE)):
            packed[e, proj] = encode(m, "q4_group128")
    for e in range(64):
        for proj in ("gate_proj", "up_proj", "down_proj"):
            pack.add_packed(expert_tensor_name(0, e, proj), packed[e % 8, proj])
    backend = native_backend.install_mixed_target_backend()
    handle = custom_op.register_expert_pack(pack)
    yield backend, handle
    custom_op.unregister_expert_pack(handle)


def _routes(tokens: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.randperm(64, generator=g)[:8] for _ in range(tokens)])
    w = torch.rand((tokens, 8), generator=g) + 0.05
    return idx.to(DEV), (w / w.sum(-1, keepdim=True)).to(DEV)


def test_two_threads_on_two_streams_get_the_serial_results(olmoe_pack):
    """Each thread has its own stream and therefore its own workspaces; prefill (64 tokens) and decode (1 token)
    calls overlap on the device and must give the bits of the same calls made one after the other."""
    _backend, handle = olmoe_pack
    cases = []
    for t in range(2):
        x = syn.activations(SEED + 10 + t, 64).to(DEV)
        idx, w = _routes(64, SEED + t)
        cases.append((x, idx, w))
    serial = [(torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True),
               torch.ops.uma_qmoe.moe_forward(x[:1], idx[:1], w[:1], 0, handle, True)) for x, idx, w in cases]
    torch.cuda.synchronize()
    results: list = [None, None]
    errors: list = []
    start = threading.Barrier(2)

    def worker(t: int) -> None:
        try:
            x, idx, w = cases[t]
            stream = torch.cuda.Stream(device=DEV)
            start.wait(timeout=60)
            with torch.cuda.stream(stream):
                outs = []
                for _ in range(20):
                    outs.append((torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True),
                                 torch.ops.uma_qmoe.moe_forward(x[:1], idx[:1], w[:1], 0, handle, True)))
            stream.synchronize()
            results[t] = outs
        except Exception as exc:                     # surfaced in the main thread
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join(timeout=300)
    assert not errors, errors
    for t in range(2):
        for many, one in results[t]:
            assert torch.equal(many, serial[t][0]) and torch.equal(one, serial[t][1])


def test_an_invalid_expert_index_is_reported_by_the_next_call_and_only_once(olmoe_pack):
    """The kernels skip a route with an out-of-range expert (the reference's kernels do the same) and record it; the
    host learns of it without waiting: the next call on the same stream and shape, or cache_summary(), raises the
    reference's message for that input, once."""
    backend, handle = olmoe_pack
    x = syn.activations(SEED + 20, 4).to(DEV)
    idx, w = _routes(4, SEED + 20)
    good = torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True)
    bad_idx = idx.clone()
    bad_idx[2, 3] = 64
    got = torch.ops.uma_qmoe.moe_forward(x, bad_idx, w, 0, handle, True)        # returns: the route contributed nothing
    torch.cuda.synchronize()
    assert torch.equal(got[:2], good[:2]) and torch.equal(got[3], good[3])
    with pytest.raises(RuntimeError, match="expert_indices contains an invalid expert"):
        torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True)
    again = torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True)          # reported once, state is clean again
    assert torch.equal(again, good)
    # the decode kernels, reported through cache_summary()
    torch.ops.uma_qmoe.moe_forward(x[:1], bad_idx[2:3], w[:1], 0, handle, True)
    with pytest.raises(RuntimeError, match="expert_indices contains an invalid expert"):
        backend.cache_summary()
    assert backend.cache_summary()["dequantized_weight_bytes"] == 0


def test_bf16_routing_weights_are_accepted(olmoe_pack):
    """The reference's CUDA back end hands BF16 routing weights to its kernels; here any floating dtype is taken and
    used as float32."""
    _backend, handle = olmoe_pack
    x = syn.activations(SEED + 30, 8).to(DEV)
    idx, w = _routes(8, SEED + 30)
    wb = w.to(torch.bfloat16)
    a = torch.ops.uma_qmoe.moe_forward(x, idx, wb, 0, handle, True)
    b = torch.ops.uma_qmoe.moe_forward(x, idx, wb.float(), 0, handle, True)
    assert torch.equal(a, b)
    assert_parity(a.cpu(), torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True).cpu(), max_abs=6e-2, cosine=0.999)
