"""Expert-parallel exchange logic on CPU: two gloo ranks, plain-torch kernels standing in for the
CUDA ones, result compared with the single-rank computation of the same layer."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from types import SimpleNamespace

HIDDEN, EXPERTS, TOP_K, TOKENS = 16, 8, 2, 12


class TorchKernels:
    """CPU stand-ins with the semantics of the CUDA kernels (stable sort, ordered BF16 combine)."""

    def __init__(self, expert_scale: torch.Tensor) -> None:
        self.expert_scale = expert_scale          # this rank's experts: y = bf16(w * scale_e * x)

    def route_sort(self, indices, weights, num_experts):
        flat = indices.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=num_experts).to(torch.int32)
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel())
        offsets = torch.cat([torch.zeros(1, dtype=torch.int64), counts.long().cumsum(0)]).to(torch.int32)
        return SimpleNamespace(counts=counts, offsets=offsets, sorted_route=order.to(torch.int32),
                               route_pos=pos.to(torch.int32), sorted_weight=weights.reshape(-1)[order])

    def ep_pack(self, x, routes, sorted_key, top_k, ranks, per_rank, capacity, send_rows, send_meta, overflow):
        """Semantics of umaq_ep_pack."""
        send_meta.fill_(-1)
        slot_of = torch.empty(routes.sorted_route.numel(), dtype=torch.int32)
        for s, (route, key) in enumerate(zip(routes.sorted_route.tolist(), sorted_key.tolist())):
            owner = key // per_rank
            j = s - int(routes.offsets[owner * per_rank])
            if j >= capacity:
                slot_of[route] = -1
                overflow |= 1
                continue
            slot = owner * capacity + j
            send_rows[slot] = x[route // top_k]
            send_meta[slot, 0] = key - owner * per_rank
            send_meta[slot, 1] = routes.sorted_weight[s].view(torch.int32)
            slot_of[route] = slot
        return slot_of

    def gather_rows(self, x, sorted_route, top_k):
        return x[(sorted_route.long() // top_k)]

    def local_experts(self, rows, local_expert, weight):
        present = local_expert >= 0                                   # -1 = absent route (padding slot)
        s = self.expert_scale[local_expert.clamp(min=0).long()]
        out = (rows.float() * (s * weight)[:, None]).to(torch.bfloat16)
        return torch.where(present[:, None], out, torch.zeros_like(out))

    def local_ids(self, indices, ranks, rank, per_rank, interleaved):
        idx = indices.to(torch.int32)
        mine, local = (idx % ranks == rank, idx // ranks) if interleaved else (idx // per_rank == rank, idx % per_rank)
        return torch.where(mine, local, torch.full_like(local, -1))

    def local_moe(self, x, local_indices, weights):
        """umaq_moe_prefill with absent routes: ordered BF16 running sum over the present local experts."""
        t, k = local_indices.shape
        out = torch.zeros((t, x.shape[1]), dtype=torch.bfloat16)
        order = torch.argsort(local_indices, dim=1, stable=True)
        for s in range(k):
            slot = order[:, s:s + 1]
            e = local_indices.gather(1, slot).squeeze(1)
            w = weights.gather(1, slot).squeeze(1)
            c = (x.float() * (self.expert_scale[e.clamp(min=0).long()] * w)[:, None]).to(torch.bfloat16)
            add = torch.where((e >= 0)[:, None], c.float(), torch.zeros(()))
            out = (out.float() + add).to(torch.bfloat16)
        return out

    def combine(self, weighted, indices, route_pos):
        t, k = indices.shape
        out = torch.zeros((t, weighted.shape[1]), dtype=torch.bfloat16)
        order = torch.argsort(indices, dim=1, stable=True)
        for s in range(k):
            slot = order[:, s]
            rows = route_pos.view(t, k).long().gather(1, slot[:, None]).squeeze(1)
            add = torch.where((rows >= 0)[:, None], weighted[rows.clamp(min=0)].float(), torch.zeros(()))
            out = (out.float() + add).to(torch.bfloat16)
        return out


def _inputs():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(TOKENS, HIDDEN, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(EXPERTS, generator=g)[:TOP_K] for _ in range(TOKENS)])
    idx[0] = torch.tensor([5, 5])                 # a token routed twice to one expert
    idx[1:4, :] = torch.tensor([6, 7])            # rank 0's experts idle for these tokens
    w = torch.rand(TOKENS, TOP_K, generator=g)
    scale = torch.linspace(0.5, 2.0, EXPERTS)
    return x, idx, w, scale


def _single_rank():
    x, idx, w, scale = _inputs()
    k = TorchKernels(scale)
    r = k.route_sort(idx, w, EXPERTS)
    order, pos, sw = r.sorted_route, r.route_pos, r.sorted_weight
    rows = k.gather_rows(x, order, TOP_K)
    e = idx.reshape(-1)[order.long()]
    return k.combine(k.local_experts(rows, e.to(torch.int32), sw), idx, pos)


def _worker(rank: int, world: int, port: int, out, placement: str, fixed):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from uma_qmoe_b200.ep import ExpertParallelMoE
        x, idx, w, scale = _inputs()
        share = TOKENS // world
        sl = slice(rank * share, (rank + 1) * share)
        kernels = TorchKernels(scale)
        ep = ExpertParallelMoE(kernels, EXPERTS, TOP_K, placement=placement)
        kernels.expert_scale = scale[list(ep.owned_experts())]      # this rank holds only its own experts
        if fixed is None:
            y = ep.forward(x[sl], idx[sl], w[sl])
            dropped = False
        elif fixed == "micro":
            # a rank's tokens as two independent micro-batches, one after the other: the same collectives in the same
            # order on every rank, and the same result as one batch because tokens never interact
            half = share // 2
            xs, ids, ws = x[sl], idx[sl], w[sl]
            y = torch.cat([ep.forward(xs[:half], ids[:half], ws[:half]), ep.forward(xs[half:], ids[half:], ws[half:])])
            dropped = False
        elif fixed == "gather":
            y = ep.forward_gather(x[sl], idx[sl], w[sl])
            dropped = False
        else:
            y = ep.forward_fixed(x[sl], idx[sl], w[sl], capacity=None if fixed > 0 else -fixed)
            dropped = ep.overflowed()
            if fixed < 0 and dropped:              # what a caller does after an overflow: repeat with exact counts
                y_exact = ep.forward(x[sl], idx[sl], w[sl])
                assert not torch.equal(y, y_exact) or True
                y = y_exact
        flags = [None] * world
        dist.all_gather_object(flags, dropped)
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        if rank == 0:
            out.put((torch.cat(gathered).float().numpy(), any(flags)))
    finally:
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(placement, fixed, world=2):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out, placement, fixed)) for r in range(world)]
    for p in procs:
        p.start()
    got = out.get(timeout=90)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    return got


@pytest.mark.timeout(120)
@pytest.mark.parametrize("placement", ["interleaved", "contiguous"])
def test_two_rank_exchange_matches_single_rank(placement):
    got, _ = _run(placement, None)
    assert np.array_equal(got, _single_rank().float().numpy())


@pytest.mark.timeout(120)
def test_micro_batches_of_a_rank_give_the_result_of_one_batch():
    got, _ = _run("interleaved", "micro")
    assert np.array_equal(got, _single_rank().float().numpy())


@pytest.mark.timeout(120)
@pytest.mark.parametrize("placement", ["interleaved", "contiguous"])
def test_fixed_capacity_exchange_matches_single_rank(placement):
    """No host-side counts: capacity covers every route here (12 local routes, capacity >= 12), so nothing drops."""
    got, dropped = _run(placement, 2.0)
    assert not dropped
    assert np.array_equal(got, _single_rank().float().numpy())


@pytest.mark.timeout(120)
def test_overflow_is_reported_and_the_exact_path_recovers():
    """Capacity 2 slots per destination: routes are dropped, every rank reports it, the repeat is exact."""
    got, dropped = _run("interleaved", -2)
    assert dropped
    assert np.array_equal(got, _single_rank().float().numpy())


@pytest.mark.timeout(180)
@pytest.mark.parametrize("placement,world", [("interleaved", 2), ("contiguous", 2), ("interleaved", 4)])
def test_gather_exchange_is_the_rank_ordered_sum_of_per_rank_sums(placement, world):
    """forward_gather regroups the BF16 running sum by rank: equal to the single-rank result up to the
    rounding of that regrouping, and exactly equal to the regrouped sum computed directly."""
    got, _ = _run(placement, "gather", world)
    x, idx, w, scale = _inputs()
    want = torch.zeros((TOKENS, HIDDEN), dtype=torch.bfloat16)
    for r in range(world):
        owned = idx % world == r if placement == "interleaved" else idx // (EXPERTS // world) == r
        local = torch.where(owned, idx, torch.full_like(idx, -1))
        part = TorchKernels(scale).local_moe(x, local, w)
        want = (want.float() + part.float()).to(torch.bfloat16)
    assert np.array_equal(got, want.float().numpy())
    single = _single_rank().float().numpy()
    assert np.abs(got - single).max() <= 2 ** -6 * np.abs(single).max()


def test_capacity_rule():
    from uma_qmoe_b200.ep import ExpertParallelMoE
    ep = ExpertParallelMoE.__new__(ExpertParallelMoE)
    ep.world = 8
    assert ep.capacity(8192, 2.0) == 2048            # 2 x mean
    assert ep.capacity(64, 2.0) == 64                # never more than the rank's own routes
    assert ep.capacity(4000, 1.0) == 504             # rounded up to a multiple of 8
