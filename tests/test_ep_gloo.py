"""Expert-parallel exchange logic on CPU: two gloo ranks, plain-torch kernels standing in for the
CUDA ones, result compared with the single-rank computation of the same layer."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

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
        return counts, order.to(torch.int32), pos.to(torch.int32), weights.reshape(-1)[order]

    def gather_rows(self, x, sorted_route, top_k):
        return x[(sorted_route.long() // top_k)]

    def local_experts(self, rows, local_expert, weight):
        s = self.expert_scale[local_expert.long()]
        return (rows.float() * (s * weight)[:, None]).to(torch.bfloat16)

    def combine(self, weighted, indices, route_pos):
        t, k = indices.shape
        out = torch.zeros((t, weighted.shape[1]), dtype=torch.bfloat16)
        order = torch.argsort(indices, dim=1, stable=True)
        for s in range(k):
            slot = order[:, s]
            rows = route_pos.view(t, k).long().gather(1, slot[:, None]).squeeze(1)
            out = (out.float() + weighted[rows].float()).to(torch.bfloat16)
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
    counts, order, pos, sw = k.route_sort(idx, w, EXPERTS)
    rows = k.gather_rows(x, order, TOP_K)
    e = idx.reshape(-1)[order.long()]
    return k.combine(k.local_experts(rows, e.to(torch.int32), sw), idx, pos)


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from uma_qmoe_b200.ep import ExpertParallelMoE
        x, idx, w, scale = _inputs()
        per = EXPERTS // world
        share = TOKENS // world
        sl = slice(rank * share, (rank + 1) * share)
        ep = ExpertParallelMoE(TorchKernels(scale[rank * per:(rank + 1) * per]), EXPERTS, TOP_K)
        y = ep.forward(x[sl], idx[sl], w[sl])
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        if rank == 0:
            out.put(torch.cat(gathered).float().numpy())
    finally:
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.timeout(120)
def test_two_rank_exchange_matches_single_rank():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = out.get(timeout=90)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    want = _single_rank().float().numpy()
    assert np.array_equal(got, want)
