"""Expert-parallel layer on one GPU (a one-rank NCCL group): the fixed-capacity dispatch kernel and the
absent-route handling of sort / gather / combine, against the plain prefill entry point."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist

from tests.helpers import SEED, expert_source, stage_layer
from uma_qmoe_b200 import synthetic as syn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def one_rank_group():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device(DEV))
    yield
    dist.destroy_process_group()


def _case(tokens=200, experts=8, top_k=4):
    src = expert_source(SEED, 7, "olmoe", "q4_group128")
    layer = stage_layer({e: src(e) for e in range(experts)}, experts, 2048, 1024, "q4_group128", DEV)
    gen = torch.Generator().manual_seed(SEED + 91)
    pop = 1.0 / torch.arange(1, experts + 1, dtype=torch.float64)
    idx = torch.multinomial(pop.expand(tokens, experts), top_k, replacement=False, generator=gen)
    w = torch.rand((tokens, top_k), generator=gen, dtype=torch.float32) / top_k
    x = syn.activations(SEED + 92, tokens)
    return layer, x.to(DEV), idx.to(DEV), w.to(DEV)


def _plain(layer, x, idx, w):
    from uma_qmoe_b200 import ops
    ws = ops.prefill_workspace(layer, x.shape[0], idx.shape[1], None, torch.device(DEV))
    y = ops.moe_prefill(layer, x, idx, w, ws)
    torch.cuda.synchronize()
    assert ops.prefill_status(ws) == 0
    return y


@pytest.mark.parametrize("placement", ["interleaved", "contiguous"])
def test_both_exchange_paths_equal_the_plain_prefill(one_rank_group, placement):
    from uma_qmoe_b200.ep import CudaKernels, ExpertParallelMoE
    layer, x, idx, w = _case()
    ep = ExpertParallelMoE(CudaKernels(layer, idx.shape[1]), layer.num_experts, idx.shape[1], placement=placement)
    want = _plain(layer, x, idx, w)
    exact = ep.forward(x, idx, w)
    fixed = ep.forward_fixed(x, idx, w)
    again = ep.forward_fixed(x, idx, w)
    assert not ep.overflowed()
    gathered = ep.forward_gather(x, idx, w)      # one rank: a single partial sum, so the bits are the same too
    assert torch.equal(exact, want)
    assert torch.equal(fixed, want) and torch.equal(again, want)
    assert torch.equal(gathered, want)


def test_absent_routes_in_the_plain_prefill(one_rank_group):
    """Half of the routes marked absent (-1) equals the same call with those routes' weights set to zero,
    up to the sign of zero, and costs no expert work for them."""
    layer, x, idx, w = _case()
    mask = torch.rand(idx.shape, generator=torch.Generator().manual_seed(5)).to(DEV) < 0.5
    got = _plain(layer, x, torch.where(mask, idx, torch.full_like(idx, -1)), w)
    want = _plain(layer, x, idx, torch.where(mask, w, torch.zeros_like(w)))
    assert torch.equal(got.float(), want.float())


def test_padding_slots_travel_as_absent_routes(one_rank_group):
    """Capacity well above the route count: most slots are padding (expert id -1) and must not change a bit."""
    from uma_qmoe_b200.ep import CudaKernels, ExpertParallelMoE
    layer, x, idx, w = _case(tokens=37)
    ep = ExpertParallelMoE(CudaKernels(layer, idx.shape[1]), layer.num_experts, idx.shape[1])
    y = ep.forward_fixed(x, idx, w, capacity=37 * 4 + 219)
    assert not ep.overflowed()
    assert torch.equal(y, _plain(layer, x, idx, w))


def test_overflow_sets_the_flag_and_drops_only_the_extra_routes(one_rank_group):
    from uma_qmoe_b200.ep import CudaKernels, ExpertParallelMoE
    layer, x, idx, w = _case()
    ep = ExpertParallelMoE(CudaKernels(layer, idx.shape[1]), layer.num_experts, idx.shape[1])
    routes = idx.numel()
    y = ep.forward_fixed(x, idx, w, capacity=routes - 40)          # the 40 last sorted routes have no slot
    assert ep.overflowed() and not ep.overflowed()                 # reported once, then cleared
    want = _plain(layer, x, idx, w)
    changed = (y != want).any(dim=1).sum().item()
    assert 0 < changed <= 40
    assert torch.isfinite(y.float()).all()
