"""Expert-parallel execution of one MoE layer over the GPUs of one node.

The reference has no multi-GPU code; this mode exists because experts are independent units: every
rank owns E/G experts of every layer and a 1/G slice of the tokens.  Placement is ``interleaved``
(expert e lives on rank e % G as local expert e // G; the default, because routers tend to give
neighbouring expert ids similar popularity and a contiguous split then overloads one rank) or
``contiguous`` (rank r owns [r*E/G, (r+1)*E/G)).  Per layer and rank:

1. route the local tokens (fused router kernel);
2. stable-sort the local routes by the key ``owner * E/G + local id`` -- which groups them by
   destination rank and, inside a rank, by local expert -- and gather the activation rows into that
   order;
3. exchange per-rank row counts, then the rows and one 8-byte record per row (local expert id,
   routing weight) (``all_to_all_single`` over NCCL / NVLink);
4. run the grouped-GEMM pipeline on the received rows (each is one route) -> weighted BF16 rows;
5. send the rows back (the reverse all-to-all) and combine each token's routes in ascending expert
   order with a BF16 running sum -- the same order and roundings as the single-GPU path, so the
   result does not depend on G.

Three exchange schemes share the placement and the kernels:

* :meth:`ExpertParallelMoE.forward` -- exact row counts (one host read per call), routes travel one by
  one; bit-identical to the single-GPU path for any G.
* :meth:`ExpertParallelMoE.forward_fixed` -- the same routes in fixed-capacity segments, no host read.
* :meth:`ExpertParallelMoE.forward_gather` -- for dense routing (top-8 of 64 over a few ranks reaches
  every rank from almost every token): all-gather the token rows once, every rank runs its own experts
  over all tokens with the other ranks' routes marked absent (expert id -1, skipped by the sort /
  gather / combine kernels), and the per-rank partial outputs return through one equal-split
  all-to-all to be summed per token in rank order.  One row per token crosses NVLink in each direction
  instead of one per route (4x fewer bytes at G = 2, top-8), and nothing waits on the host.  The sum
  is a BF16 running sum over ranks of BF16 running sums over each rank's experts: within the path's
  tolerance of the single-GPU result, not bit-identical to it.

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
        self._ws: Optional[torch.Tensor] = None
        self._ws_rows = 0
        self._ws_moe: Optional[torch.Tensor] = None
        self._ws_moe_shape = (0, 0)

    def route_sort(self, indices: torch.Tensor, weights: torch.Tensor, num_experts: int):
        """-> object with counts, offsets, sorted_route, route_pos, sorted_weight"""
        return self.ops.route_sort(indices, weights, num_experts)

    def ep_pack(self, x: torch.Tensor, routes: Any, sorted_key: torch.Tensor, top_k: int, ranks: int, per_rank: int,
                capacity: int, send_rows: torch.Tensor, send_meta: torch.Tensor, overflow: torch.Tensor) -> torch.Tensor:
        return self.ops.ep_pack(x, routes, sorted_key, top_k, ranks, per_rank, capacity, send_rows, send_meta, overflow)

    def gather_rows(self, x: torch.Tensor, sorted_route: torch.Tensor, top_k: int) -> torch.Tensor:
        return self.ops.gather_rows(x, sorted_route, top_k, permute=False)

    def local_experts(self, rows: torch.Tensor, local_expert: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        n = rows.shape[0]
        if n == 0:
            return rows
        if self._ws_rows < n:                   # grow-only: the received row count changes every call
            self._ws_rows = n + n // 4
            self._ws = self.ops.prefill_workspace(self.layer, self._ws_rows, 1, None, rows.device)
        return self.ops.moe_prefill(self.layer, rows, local_expert.view(n, 1), weight.view(n, 1), self._ws)

    def combine(self, weighted: torch.Tensor, indices: torch.Tensor, route_pos: torch.Tensor) -> torch.Tensor:
        return self.ops.combine_routes(weighted, indices, route_pos)

    def local_ids(self, indices: torch.Tensor, ranks: int, rank: int, per_rank: int, interleaved: bool) -> torch.Tensor:
        return self.ops.ep_local_ids(indices, ranks, rank, per_rank, interleaved)

    @property
    def rows_k_permuted(self) -> bool:
        """Quantised layers read their activation rows in a permuted k order; the push can write that order."""
        return self.layer.encoding != "bf16_le"

    @property
    def push_flags(self) -> int:
        """The sender does the receiver's two preparation passes: ids local to the destination, rows in k order."""
        return self.ops.EP_LOCAL_IDS | (self.ops.EP_K_PERMUTED if self.rows_k_permuted else 0)

    def local_moe_to_peers(self, x: torch.Tensor, local_indices: torch.Tensor, weights: torch.Tensor, ex: Any) -> None:
        """Like :meth:`local_moe`, but every token's partial sum goes straight into its owner rank's buffer; ``x``
        and ``local_indices`` as :attr:`push_flags` made the senders write them."""
        n, top_k = local_indices.shape
        if self._ws_moe is None or self._ws_moe_shape != (n, top_k):
            self._ws_moe = self.ops.prefill_workspace(self.layer, n, top_k, None, x.device)
            self._ws_moe_shape = (n, top_k)
        self.ops.moe_prefill_to_peers(self.layer, x, local_indices, weights, ex.peers, ex.off_parts, ex.tokens, self._ws_moe,
                                      rows_k_permuted=self.rows_k_permuted)

    def peer_layer(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor, ex: Any, per_rank: int,
                   interleaved: bool) -> torch.Tensor:
        """The whole peer-memory layer (push, barrier, local experts + combine to the owners, barrier, final combine)
        issued by one native call: five launches' worth of host work for the price of one."""
        n, top_k = ex.tokens * ex.peers.ranks, indices.shape[1]
        if self._ws_moe is None or self._ws_moe_shape != (n, top_k):
            self._ws_moe = self.ops.prefill_workspace(self.layer, n, top_k, None, x.device)
            self._ws_moe_shape = (n, top_k)
        return self.ops.ep_layer(self.layer, x, indices, weights, per_rank, interleaved, ex, self._ws_moe)

    def local_moe(self, x: torch.Tensor, local_indices: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """This rank's experts over all rows of x; local_indices -1 = the route belongs to another rank."""
        n, top_k = local_indices.shape
        if self._ws_moe is None or self._ws_moe_shape != (n, top_k):
            self._ws_moe = self.ops.prefill_workspace(self.layer, n, top_k, None, x.device)
            self._ws_moe_shape = (n, top_k)
        return self.ops.moe_prefill(self.layer, x, local_indices, weights, self._ws_moe)


class PeerExchange:
    """One buffer per rank that every rank can address, and this rank's view of all of them.

    Layout (the same on every rank; t = tokens per rank, G ranks): rows ``[G*t, H]`` BF16, ids ``[G*t, k]``
    int32 and weights ``[G*t, k]`` float32 pushed by the ranks, ``parts [G*t, H]`` BF16 written by the ranks'
    combine kernels (row ``p*t + i`` = rank p's partial sum for local token i), and one flag word per rank for
    the barrier.  ``buffers`` may be given (one CUDA byte tensor per rank, all on one device) to run several
    ranks in one process; otherwise the buffer comes from ``torch.distributed._symmetric_memory`` and is
    mapped by all ranks of ``group``.
    """

    def __init__(self, tokens: int, hidden: int, top_k: int, rank: int, world: int, device: torch.device,
                 group: Any = None, buffers: Optional[list] = None) -> None:
        from . import ops
        align = lambda n: (n + 255) // 256 * 256
        rows = world * tokens
        self.tokens, self.hidden, self.top_k, self.rank, self.world = tokens, hidden, top_k, rank, world
        self.off_rows = 0
        self.off_ids = align(rows * hidden * 2)
        self.off_w = self.off_ids + align(rows * top_k * 4)
        self.off_parts = self.off_w + align(rows * top_k * 4)
        self.off_flags = self.off_parts + align(rows * hidden * 2)
        self.nbytes = self.off_flags + 256
        if buffers is not None:
            self.buffer = buffers[rank]
            pointers = [b.data_ptr() for b in buffers]
            self.handle = None
        else:
            import torch.distributed._symmetric_memory as symm
            self.buffer = symm.empty(self.nbytes, dtype=torch.uint8, device=device)
            self.buffer.zero_()
            self.handle = symm.rendezvous(self.buffer, dist.group.WORLD if group is None else group)
            pointers = [int(p) for p in self.handle.buffer_ptrs]
        if self.buffer.numel() < self.nbytes:
            raise RuntimeError("exchange buffer too small")
        self.peers = ops.ep_peers(pointers, rank)
        view = lambda off, n, dtype: self.buffer[off:off + n].view(dtype)
        self.all_x = view(self.off_rows, rows * hidden * 2, torch.bfloat16).view(rows, hidden)
        self.all_idx = view(self.off_ids, rows * top_k * 4, torch.int32).view(rows, top_k)
        self.all_w = view(self.off_w, rows * top_k * 4, torch.float32).view(rows, top_k)
        self.parts = view(self.off_parts, rows * hidden * 2, torch.bfloat16).view(rows, hidden)
        self.present = torch.empty((tokens, world), dtype=torch.int32, device=device)
        self.part_pos = (torch.arange(world, dtype=torch.int32, device=device)[None, :] * tokens +
                         torch.arange(tokens, dtype=torch.int32, device=device)[:, None]).contiguous()
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    @staticmethod
    def nbytes_for(tokens: int, hidden: int, top_k: int, world: int) -> int:
        align = lambda n: (n + 255) // 256 * 256
        rows = world * tokens
        return 2 * align(rows * hidden * 2) + 2 * align(rows * top_k * 4) + 256

    def timed_out(self) -> bool:
        """True if a barrier gave up waiting for a peer (synchronises)."""
        return int(self.status.item()) != 0


@dataclass
class ExchangePlan:
    send_counts: list[int]
    recv_counts: list[int]


class ExpertParallelMoE:
    def __init__(self, kernels: Any, num_experts: int, top_k: int, group: Optional[dist.ProcessGroup] = None,
                 placement: str = "interleaved", world: Optional[int] = None, rank: Optional[int] = None) -> None:
        """``world`` / ``rank`` default to the process group's; given explicitly they let one process stand for
        several ranks (only the peer-memory exchange, which needs no collective, can be driven that way)."""
        if placement not in ("interleaved", "contiguous"):
            raise RuntimeError(f"unknown expert placement {placement!r}")
        self.placement = placement
        self._keys: Optional[torch.Tensor] = None
        self._fixed: Optional[tuple] = None
        self._gather: Optional[tuple] = None
        self._overflow: Optional[torch.Tensor] = None
        self.kernels = kernels
        self.group = group
        self.world = dist.get_world_size(group) if world is None else world
        self.rank = dist.get_rank(group) if rank is None else rank
        if num_experts % self.world:
            raise RuntimeError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts = num_experts
        self.per_rank = num_experts // self.world
        self.top_k = top_k

    def owned_experts(self, rank: Optional[int] = None) -> range:
        """Global ids of the experts rank ``rank`` holds, in local-id order."""
        r = self.rank if rank is None else rank
        if self.placement == "interleaved":
            return range(r, self.num_experts, self.world)
        return range(r * self.per_rank, (r + 1) * self.per_rank)

    def sort_keys(self, indices: torch.Tensor) -> torch.Tensor:
        """owner * E/G + local id of every selected expert (the identity for contiguous placement)."""
        if self.placement == "contiguous":
            return indices
        if self._keys is None or self._keys.device != indices.device:
            e = torch.arange(self.num_experts, device=indices.device)
            self._keys = ((e % self.world) * self.per_rank + e // self.world).to(torch.int64)
        return self._keys[indices.long()].to(indices.dtype)

    def capacity(self, local_routes: int, factor: float) -> int:
        """Slots per (source, destination) pair of the fixed-capacity exchange."""
        mean = -(-local_routes // self.world)
        cap = min(local_routes, max(128, int(factor * mean)))
        return -(-cap // 8) * 8

    def overflowed(self) -> bool:
        """True if any fixed-capacity call since the last query dropped a route (synchronises)."""
        if self._overflow is None:
            return False
        hit = bool(self._overflow.item())
        self._overflow.zero_()
        return hit

    def forward_fixed(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                      capacity_factor: float = 2.0, capacity: Optional[int] = None) -> torch.Tensor:
        """Same result as :meth:`forward` without any host synchronisation: every (source, destination)
        pair exchanges ``capacity`` slots, unused slots travel as absent routes (expert id -1) and are
        skipped by the sort / gather / combine kernels.  If a destination gets more than ``capacity``
        routes from this rank the extra routes are dropped and :meth:`overflowed` reports it; the caller
        then repeats the step with :meth:`forward`."""
        k = self.kernels
        t, top_k = indices.shape
        routes = t * top_k
        cap = self.capacity(routes, capacity_factor) if capacity is None else capacity
        slots = self.world * cap
        if self._fixed is None or self._fixed[0].shape[0] != slots or self._fixed[0].device != x.device:
            self._fixed = (x.new_empty((slots, x.shape[1])), torch.empty((slots, 2), dtype=torch.int32, device=x.device),
                           x.new_empty((slots, x.shape[1])), torch.empty((slots, 2), dtype=torch.int32, device=x.device),
                           x.new_empty((slots, x.shape[1])))
            self._overflow = torch.zeros(1, dtype=torch.int32, device=x.device)
        send_rows, send_meta, recv_rows, recv_meta, back = self._fixed
        keys = self.sort_keys(indices)
        r = k.route_sort(keys, weights, self.num_experts)
        sorted_key = keys.reshape(-1).index_select(0, r.sorted_route.long()).to(torch.int32)
        route_slot = k.ep_pack(x, r, sorted_key, top_k, self.world, self.per_rank, cap, send_rows, send_meta,
                               self._overflow)
        dist.all_to_all_single(recv_rows, send_rows, group=self.group)
        dist.all_to_all_single(recv_meta, send_meta, group=self.group)
        done = k.local_experts(recv_rows, recv_meta[:, 0].contiguous(), recv_meta[:, 1].contiguous().view(torch.float32))
        dist.all_to_all_single(back, done, group=self.group)
        return k.combine(back, indices, route_slot)

    def forward_gather(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """All-gather the rows, run the local experts over all of them, all-to-all the partial sums back."""
        k = self.kernels
        t, top_k = indices.shape
        g = self.world
        if self._gather is None or self._gather[0].shape[0] != g * t or self._gather[0].device != x.device:
            self._gather = (x.new_empty((g * t, x.shape[1])),
                            (torch.empty((g * t, top_k), dtype=indices.dtype, device=x.device),
                             torch.empty((g * t, top_k), dtype=torch.float32, device=x.device)),
                            x.new_empty((g * t, x.shape[1])),
                            torch.arange(g, dtype=torch.int32, device=x.device).repeat(t, 1).contiguous(),
                            (torch.arange(g, dtype=torch.int32, device=x.device)[None, :] * t +
                             torch.arange(t, dtype=torch.int32, device=x.device)[:, None]).contiguous())
        all_x, (all_idx, all_w), parts, rank_ids, part_pos = self._gather
        dist.all_gather_into_tensor(all_x, x.contiguous(), group=self.group)
        dist.all_gather_into_tensor(all_idx, indices.contiguous(), group=self.group)
        dist.all_gather_into_tensor(all_w, weights.contiguous(), group=self.group)
        local = k.local_ids(all_idx, g, self.rank, self.per_rank, self.placement == "interleaved")
        partial = k.local_moe(all_x, local, all_w)
        dist.all_to_all_single(parts, partial, group=self.group)      # parts[r * t + i] = rank r's sum for my token i
        return k.combine(parts, rank_ids, part_pos)

    # ---- exchange over peer memory: no collective library on the data path --------------------------------
    def peer_push(self, ex: PeerExchange, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor) -> None:
        """Phase 1: this rank's rows (to the ranks that own one of the token's experts) and routes (to all)."""
        self.kernels.ops.ep_push(x, indices, weights, self.per_rank, self.placement == "interleaved", ex.peers,
                                 ex.off_rows, ex.off_ids, ex.off_w, ex.present, flags=self.kernels.push_flags)

    def peer_compute(self, ex: PeerExchange) -> None:
        """Phase 2: this rank's experts over everything that was pushed to it; the combine writes every token's
        partial sum into its owner's buffer."""
        self.kernels.local_moe_to_peers(ex.all_x, ex.all_idx, ex.all_w, ex)     # the ids arrived local to this rank

    def peer_combine(self, ex: PeerExchange) -> torch.Tensor:
        """Phase 3: the partial sums of the ranks that worked on a token, added in rank order."""
        return self.kernels.combine(ex.parts, ex.present, ex.part_pos)

    def forward_peer(self, ex: PeerExchange, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """Same result contract as :meth:`forward_gather`, with the two exchanges done by this library's own
        kernels over peer memory: rows travel only to ranks that own one of the token's experts, partial sums
        only back from ranks that did some work, and the only synchronisation is a flag barrier per phase."""
        if hasattr(self.kernels, "peer_layer") and x.is_contiguous() and indices.is_contiguous() and weights.is_contiguous():
            return self.kernels.peer_layer(x, indices, weights, ex, self.per_rank, self.placement == "interleaved")
        ops = self.kernels.ops
        self.peer_push(ex, x, indices, weights)
        ops.ep_barrier(ex.peers, ex.off_flags, ex.epoch, ex.status)
        self.peer_compute(ex)
        ops.ep_barrier(ex.peers, ex.off_flags, ex.epoch, ex.status)
        return self.peer_combine(ex)

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
        keys = self.sort_keys(indices)
        r = k.route_sort(keys, weights, self.num_experts)
        counts, sorted_route, route_pos, sorted_weight = r.counts, r.sorted_route, r.route_pos, r.sorted_weight
        # queue the device work that does not need the counts before the host waits for them
        send_rows = k.gather_rows(x, sorted_route, self.top_k)
        # one record per sorted route: local expert id (key modulo E/G) and the float32 routing weight
        sorted_key = keys.reshape(-1).index_select(0, sorted_route.long())
        local_expert = (sorted_key % self.per_rank).to(torch.int32)
        meta = torch.stack((local_expert, sorted_weight.contiguous().view(torch.int32)), dim=1)
        plan = self.plan(counts)
        n_recv = sum(plan.recv_counts)
        recv_rows = self._exchange(n_recv, send_rows, plan.recv_counts, plan.send_counts)
        recv_meta = self._exchange(n_recv, meta, plan.recv_counts, plan.send_counts)
        recv_expert = recv_meta[:, 0].contiguous()
        recv_weight = recv_meta[:, 1].contiguous().view(torch.float32)
        done = k.local_experts(recv_rows, recv_expert, recv_weight)
        back = self._exchange(send_rows.shape[0], done, plan.send_counts, plan.recv_counts)
        return k.combine(back, indices, route_pos)
