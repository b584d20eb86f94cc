"""Device-resident synthetic MoE layers and the layer stack the benchmarks step through.

Weights are generated on the GPU from a seed (N(0, 0.02) in BF16) and packed by the device-side
packer into the canonical bytes, so a 16-layer OLMoE-shaped stack (3.4 GB of Q4) is ready in well
under a second; nothing here reads a checkpoint.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import ops
from .ops import DeviceLayer, DeviceSharedExpert
from .synthetic import ModelShape, router_weight


def balanced_order(router: torch.Tensor, ranks: int) -> list[int]:
    """A relabelling of the experts for expert parallelism: position n of the result is the expert that gets the
    new id n, chosen so that the interleaved placement (new id n on rank n % ranks) spreads the expected load
    evenly.  The load estimate is static and needs no data: an expert's logit scales with the norm of its router
    row, so rows are ranked by norm and dealt to the ranks in serpentine order.  Relabelling changes nothing about
    the model (the router rows move with the experts)."""
    norms = router.float().norm(dim=1)
    by_load = torch.argsort(norms, descending=True).tolist()
    per_rank: list[list[int]] = [[] for _ in range(ranks)]
    for i, e in enumerate(by_load):
        lap, pos = divmod(i, ranks)
        per_rank[pos if lap % 2 == 0 else ranks - 1 - pos].append(e)
    order = [0] * len(by_load)
    for r, mine in enumerate(per_rank):
        for j, e in enumerate(mine):
            order[j * ranks + r] = e
    return order


def random_layer(shape: ModelShape, encoding: str, seed: int, device: torch.device,
                 experts: Optional[Sequence[int]] = None) -> DeviceLayer:
    """One layer of `shape` with experts `experts` (default: all, in id order) in `encoding`."""
    experts = range(shape.experts) if experts is None else experts
    gen = torch.Generator(device=device)
    n = len(experts)

    def projection(tag: int, rows: int, k: int):
        # every expert's weights depend only on (seed, projection, GLOBAL expert id): a rank that holds a
        # subset of the experts holds exactly the bytes the full layer has for them
        w = torch.empty(n * rows * k, device=device, dtype=torch.bfloat16)
        for j, e in enumerate(experts):
            gen.manual_seed(seed * 1000003 + tag * 7919 + e * 104729)
            w[j * rows * k:(j + 1) * rows * k] = (
                torch.randn(rows * k, device=device, generator=gen, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        if encoding == "bf16_le":
            return w.view(torch.uint8), None
        return ops.quantize_groups(w, encoding)

    g, gs = projection(0, shape.intermediate, shape.hidden)
    u, us = projection(1, shape.intermediate, shape.hidden)
    d, ds = projection(2, shape.hidden, shape.intermediate)
    return DeviceLayer(encoding, n, shape.hidden, shape.intermediate, g, u, d, gs, us, ds)


def random_shared_expert(shape: ModelShape, seed: int, device: torch.device) -> DeviceSharedExpert:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 1000003 + 99991)
    s, h = shape.shared_intermediate, shape.hidden
    mk = lambda *dims: (torch.randn(*dims, device=device, generator=gen) * 0.02).to(torch.bfloat16)
    return DeviceSharedExpert(mk(s, h), mk(s, h), mk(h, s), mk(1, h))


def rms_renorm(x: torch.Tensor) -> torch.Tensor:
    """Keeps the activations at unit RMS from layer to layer (there is no attention or norm between
    the MoE layers of the synthetic stack)."""
    return torch.nn.functional.rms_norm(x, (x.shape[-1],), None, 1e-6)


@dataclass
class MoEStack:
    shape: ModelShape
    layers: list[DeviceLayer]
    routers: list[torch.Tensor]
    renormalize: bool
    orders: Optional[list] = None      # per layer: original expert id behind every (new) id

    @classmethod
    def build(cls, shape: ModelShape, encoding: str, num_layers: int, seed: int, device: torch.device,
              renormalize: bool, skew: float = 1.0, experts: Optional[Sequence[int]] = None,
              balance_ranks: int = 0) -> "MoEStack":
        """``experts``: the (new) expert ids this rank holds, default all.  ``balance_ranks`` > 1 relabels the
        experts of every layer with :func:`balanced_order` first; ``orders[l][n]`` is then the original expert
        behind new id n (the weights of an expert depend only on its original id and the seeds)."""
        routers, layers, orders = [], [], []
        for l in range(num_layers):
            wr = router_weight(seed, l, shape, skew=skew)
            order = balanced_order(wr, balance_ranks) if balance_ranks > 1 else list(range(shape.experts))
            held = order if experts is None else [order[n] for n in experts]
            routers.append(wr[order].contiguous().to(device))
            layers.append(random_layer(shape, encoding, seed + l, device, held))
            orders.append(order)
        stack = cls(shape, layers, routers, renormalize)
        stack.orders = orders
        return stack

    def route(self, layer: int, x: torch.Tensor):
        return ops.route_topk(x, self.routers[layer], self.shape.top_k, self.renormalize)

    @property
    def device_bytes(self) -> int:
        return sum(l.device_storage_bytes for l in self.layers)
