"""Expert-parallel execution of one MoE layer over the GPUs of one node.

The reference has no multi-GPU code; this mode exists because experts are independent units: rank r
owns the contiguous experts [r*E/G, (r+1)*E/G) of every layer and a 1/G slice of the tokens.  Per
layer and rank:

1. route the local tokens (fused router kernel);
2. stable-sort the local routes by global expert id -- which also groups them by destination rank,
   since ranks own contiguous expert ranges -- and gather the activation rows into that order;
3. exchange per-rank row counts, then the rows with their local expert id and routing weight
   (``all_to_all_single`` over NCCL / NVLink);
4. run the grouped-GEMM pipeline on the received rows (each is one route) -> weighted BF16 rows;
5. send the rows back (the reverse all-to-all) and combine each token's routes in ascending expert
   order with a BF16 running sum -- the same order and roundings as the single-GPU path, so the
   result does not depend on G.

Everything that touches tensors goes through a ``kernels`` object; the default drives the CUDA
kernels, the CPU tests substitute plain torch functions to exercise the exchange logic over gloo.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.distributed as dist


class CudaKernels:
    """The product path: every step is one of the library's kernels."""

    def __init__(self, layer: Any, top_k: int) -> None:
        from . import ops
        self.ops = ops
        self.layer = layer                      # DeviceLayer holding only this rank's experts
        self.top_k = top_k
        self._ws: dict[int, torch.Tensor] = {}

    def route_sort(self, indices: torch.Tensor, weights: torch.Tensor, num_experts: int):
        r = self.ops.route_sort(indices, weights, num_experts)
        return r.counts, r.sorted_route, r.route_pos, r.sorted_weight

    def gather_rows(self, x: torch.Tensor, sorted_route: torch.Tensor, top_k: int) -> torch.Tensor:
        return self.ops.gather_rows(x, sorted_route, top_k, permute=False)

    def local_experts(self, rows: torch.Tensor, local_expert: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        n = rows.shape[0]
        if n == 0:
            return rows
        ws = self._ws.get(n)
        if ws is None:
            self._ws.clear()
            ws = self._ws[n] = self.ops.prefill_workspace(self.layer, n, 1, None, rows.device)
        return self.ops.moe_prefill(self.layer, rows, local_expert.view(n, 1), weight.view(n, 1), ws)

    def combine(self, weighted: torch.Tensor, indices: torch.Tensor, route_pos: torch.Tensor) -> torch.Tensor:
        return self.ops.combine_routes(weighted, indices, route_pos)


@dataclass
class ExchangePlan:
    send_counts: list[int]
    recv_counts: list[int]


class ExpertParallelMoE:
    def __init__(self, kernels: Any, num_experts: int, top_k: int, group: Optional[dist.ProcessGroup] = None) -> None:
        self.kernels = kernels
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise RuntimeError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts = num_experts
        self.per_rank = num_experts // self.world
        self.top_k = top_k

    def plan(self, counts: torch.Tensor) -> ExchangePlan:
        """Rows this rank sends to / receives from every rank (one small collective + one host read)."""
        send = counts.view(self.world, self.per_rank).sum(dim=1).to(torch.int64)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        both = torch.stack((send, recv)).cpu()
        return ExchangePlan(both[0].tolist(), both[1].tolist())

    def _exchange(self, out_rows: int, tensor: torch.Tensor, out_splits: list[int], in_splits: list[int]) -> torch.Tensor:
        out = tensor.new_empty((out_rows, *tensor.shape[1:]))
        dist.all_to_all_single(out, tensor, out_splits, in_splits, group=self.group)
        return out

    def forward(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """x [t, H] local tokens, indices/weights [t, k] over the GLOBAL experts -> [t, H]."""
        k = self.kernels
        counts, sorted_route, route_pos, sorted_weight = k.route_sort(indices, weights, self.num_experts)
        plan = self.plan(counts)
        send_rows = k.gather_rows(x, sorted_route, self.top_k)
        # local expert id of every sorted route: global id minus the owner's first expert
        sorted_expert = indices.reshape(-1).index_select(0, sorted_route.long())
        local_expert = (sorted_expert % self.per_rank).to(torch.int32)
        n_recv = sum(plan.recv_counts)
        recv_rows = self._exchange(n_recv, send_rows, plan.recv_counts, plan.send_counts)
        recv_expert = self._exchange(n_recv, local_expert, plan.recv_counts, plan.send_counts)
        recv_weight = self._exchange(n_recv, sorted_weight, plan.recv_counts, plan.send_counts)
        done = k.local_experts(recv_rows, recv_expert, recv_weight)
        back = self._exchange(send_rows.shape[0], done, plan.send_counts, plan.recv_counts)
        return k.combine(back, indices, route_pos)
