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


# ---- exchange over peer memory ------------------------------------------------------------------------------

def _rank_layers(ranks, placement, experts=8):
    """The full layer and every rank's slice of it (the same expert bytes)."""
    src = expert_source(SEED, 7, "olmoe", "q4_group128")
    full = stage_layer({e: src(e) for e in range(experts)}, experts, 2048, 1024, "q4_group128", DEV)
    per = experts // ranks
    owned = [list(range(r, experts, ranks)) if placement == "interleaved" else list(range(r * per, (r + 1) * per))
             for r in range(ranks)]
    slices = [stage_layer({i: src(e) for i, e in enumerate(own)}, per, 2048, 1024, "q4_group128", DEV) for own in owned]
    return full, slices


@pytest.mark.parametrize("ranks,placement", [(2, "interleaved"), (4, "interleaved"), (4, "contiguous")])
def test_peer_exchange_with_every_rank_on_one_gpu(ranks, placement):
    """The push / compute / combine kernels of the peer-memory exchange, with all ranks' buffers on one device and
    the phases run rank after rank (no barrier kernel: the loop order is the barrier).  Buffers start as NaN
    patterns, so a row that was not pushed, or a partial sum that was not written, would poison the result."""
    from uma_qmoe_b200 import ops
    from uma_qmoe_b200.ep import CudaKernels, ExpertParallelMoE, PeerExchange
    top_k, t = 4, 50
    full, slices = _rank_layers(ranks, placement)
    gen = torch.Generator().manual_seed(SEED + 93)
    pop = 1.0 / torch.arange(1, 9, dtype=torch.float64)
    idx = torch.multinomial(pop.expand(ranks * t, 8), top_k, replacement=False, generator=gen).to(DEV)
    w = (torch.rand((ranks * t, top_k), generator=gen, dtype=torch.float32) / top_k).to(DEV)
    x = syn.activations(SEED + 94, ranks * t).to(DEV)
    want = _plain(full, x, idx, w)
    nbytes = PeerExchange.nbytes_for(t, 2048, top_k, ranks)
    buffers = [torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=DEV) for _ in range(ranks)]
    eps, exs = [], []
    for r in range(ranks):
        eps.append(ExpertParallelMoE(CudaKernels(slices[r], top_k), 8, top_k, placement=placement, world=ranks, rank=r))
        exs.append(PeerExchange(t, 2048, top_k, r, ranks, torch.device(DEV), buffers=buffers))
    rows = lambda r: slice(r * t, (r + 1) * t)
    for r in range(ranks):
        eps[r].peer_push(exs[r], x[rows(r)].contiguous(), idx[rows(r)].contiguous(), w[rows(r)].contiguous())
    for r in range(ranks):
        eps[r].peer_compute(exs[r])
    got = torch.cat([eps[r].peer_combine(exs[r]) for r in range(ranks)])
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
    # a BF16 sum over ranks of BF16 ordered sums: inside the operator's tolerance of the one-GPU result, not bit-equal
    from oracle import moe_oracle as orc
    m = orc.compare(got.cpu(), want.cpu())
    assert m["max_abs"] <= 2e-2 and m["cosine"] >= 0.9999, m
    # the table of who holds part of a token: rank p is present iff it owns one of the token's experts
    owner = (idx % ranks) if placement == "interleaved" else (idx // (8 // ranks))
    for r in range(ranks):
        expect = torch.stack([(owner[rows(r)] == p).any(dim=1) for p in range(ranks)], dim=1)
        assert torch.equal(exs[r].present >= 0, expect)


@pytest.mark.parametrize("placement", ["interleaved", "contiguous"])
def test_push_prepares_the_receivers_input(placement):
    """With UMAQ_EP_LOCAL_IDS | UMAQ_EP_K_PERMUTED the id table a rank receives equals what ``ep_local_ids`` makes of
    the global ids there, and the rows it receives equal the k-permutation ``gather_rows`` makes of the senders' rows;
    without the flags both arrive unchanged.  Rows of tokens with no expert on the rank are not pushed."""
    from uma_qmoe_b200 import ops
    from uma_qmoe_b200.ep import PeerExchange
    ranks, top_k, t, experts = 4, 4, 37, 8
    per = experts // ranks
    gen = torch.Generator().manual_seed(SEED + 211)
    idx = torch.multinomial(torch.ones(ranks * t, experts), top_k, replacement=False, generator=gen).to(torch.int32).to(DEV)
    idx[5, 1] = -1                                              # an absent route stays absent everywhere
    w = torch.rand((ranks * t, top_k), generator=gen, dtype=torch.float32).to(DEV)
    x = syn.activations(SEED + 212, ranks * t).to(DEV)
    nbytes = PeerExchange.nbytes_for(t, 2048, top_k, ranks)
    for flags in (0, ops.EP_LOCAL_IDS | ops.EP_K_PERMUTED):
        buffers = [torch.full((nbytes,), 0xFF, dtype=torch.uint8, device=DEV) for _ in range(ranks)]
        exs = [PeerExchange(t, 2048, top_k, r, ranks, torch.device(DEV), buffers=buffers) for r in range(ranks)]
        for r in range(ranks):
            rows = slice(r * t, (r + 1) * t)
            ops.ep_push(x[rows].contiguous(), idx[rows].contiguous(), w[rows].contiguous(), per, placement == "interleaved",
                        exs[r].peers, exs[r].off_rows, exs[r].off_ids, exs[r].off_w, exs[r].present, flags=flags)
        torch.cuda.synchronize()
        x_want = ops.gather_rows(x, None, 1, permute=True) if flags else x
        for p in range(ranks):
            local = ops.ep_local_ids(idx, ranks, p, per, placement == "interleaved")
            assert torch.equal(exs[p].all_idx, local if flags else idx)
            assert torch.equal(exs[p].all_w, w)
            pushed = (local >= 0).any(dim=1)
            assert torch.equal(exs[p].all_x[pushed], x_want[pushed])
            assert (exs[p].all_x[~pushed].view(torch.int16) == -1).all()      # never written: still the fill pattern


def test_layer_call_with_one_rank_equals_the_plain_prefill():
    """``umaq_ep_layer`` (push, barrier, local experts, barrier, final combine from one native call) with a single
    rank: every route is local, the barriers signal and wait for the rank's own flag word, and a one-term BF16 sum is
    the plain operator's result bit for bit.  Called twice: the epoch counts on, nothing is reset between layers."""
    from uma_qmoe_b200.ep import CudaKernels, ExpertParallelMoE, PeerExchange
    full, _ = _rank_layers(1, "interleaved")
    top_k, t = 4, 70
    gen = torch.Generator().manual_seed(SEED + 307)
    idx = torch.multinomial(torch.ones(t, 8), top_k, replacement=False, generator=gen).to(DEV)
    w = (torch.rand((t, top_k), generator=gen, dtype=torch.float32) / top_k).to(DEV)
    x = syn.activations(SEED + 308, t).to(DEV)
    want = _plain(full, x, idx, w)
    buffers = [torch.full((PeerExchange.nbytes_for(t, 2048, top_k, 1),), 0xFF, dtype=torch.uint8, device=DEV)]
    buffers[0][-256:] = 0                                       # the flag words start at zero
    ex = PeerExchange(t, 2048, top_k, 0, 1, torch.device(DEV), buffers=buffers)
    ep = ExpertParallelMoE(CudaKernels(full, top_k), 8, top_k, world=1, rank=0)
    for _ in range(2):
        got = ep.forward_peer(ex, x, idx, w)
        torch.cuda.synchronize()
        assert not ex.timed_out()
        assert torch.equal(got, want)
    assert int(ex.epoch.item()) == 4


def _peer_worker(rank, world, port, results):
    import traceback
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from oracle import moe_oracle as orc
        from uma_qmoe_b200 import ops
        from uma_qmoe_b200.ep import CudaKernels, ExpertParallelMoE, PeerExchange
        from uma_qmoe_b200.stack import random_layer
        shape, t = syn.OLMOE, 256
        mine = range(rank, shape.experts, world)
        layer = random_layer(shape, "q4_group128", SEED, dev, mine)
        full = random_layer(shape, "q4_group128", SEED, dev)
        x_all = syn.activations(SEED + 95, world * t).to(dev)
        wr = syn.router_weight(SEED, 0, shape, skew=1.0).to(dev)
        w_all, idx_all = ops.route_topk(x_all, wr, shape.top_k, True)
        mine_rows = slice(rank * t, (rank + 1) * t)
        x, w, idx = x_all[mine_rows].contiguous(), w_all[mine_rows].contiguous(), idx_all[mine_rows].contiguous()
        ws = ops.prefill_workspace(full, t, shape.top_k, None, dev)
        want = ops.moe_prefill(full, x, idx, w, ws)
        ep = ExpertParallelMoE(CudaKernels(layer, shape.top_k), shape.experts, shape.top_k)
        out = {"exact_equal": bool(torch.equal(ep.forward(x, idx, w), want))}
        out["gather"] = orc.compare(ep.forward_gather(x, idx, w).cpu(), want.cpu())
        try:
            ex = PeerExchange(t, shape.hidden, shape.top_k, rank, world, dev)
            dist.barrier()
            for _ in range(2):                               # twice: the second call reuses every buffer
                got = ep.forward_peer(ex, x, idx, w)
            torch.cuda.synchronize()
            out["peer"] = orc.compare(got.cpu(), want.cpu())
            out["peer_timed_out"] = ex.timed_out()
        except Exception as exc:                              # no peer mapping on this machine: say so, NCCL paths stand
            out["peer_unavailable"] = f"{type(exc).__name__}: {exc}"[:200]
        results[rank] = out
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        results[rank] = {"error": traceback.format_exc()[-1500:]}


def test_two_gpu_exchanges_match_the_one_gpu_result():
    """Two real ranks: the exact-count exchange is bit-identical to the one-GPU operator, the gather exchange and the
    peer-memory exchange stay inside the operator's tolerance of it.  Needs two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_peer_worker, args=(r, 2, port, results)) for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=600)
    for r in range(2):
        out = results.get(r)
        assert out is not None and "error" not in out, out
        assert out["exact_equal"], out
        assert out["gather"]["max_abs"] <= 2e-2 and out["gather"]["cosine"] >= 0.9999, out
        if "peer" in out:
            assert not out["peer_timed_out"], out
            assert out["peer"]["max_abs"] <= 2e-2 and out["peer"]["cosine"] >= 0.9999, out
