"""Prefill path (route sort, tcgen05 grouped GEMMs, ordered combine) and the fused router vs the
CPU oracle and the reference-made golden vectors, through the C ABI."""

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.helpers import SEED, assert_parity, bits_to_bf16, expert_source, stage_layer
from uma_qmoe_b200 import synthetic as syn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_prefill(layer, x, idx, w, shared=None):
    from uma_qmoe_b200 import ops
    ws = ops.prefill_workspace(layer, x.shape[0], idx.shape[1], shared, torch.device(DEV))
    args = (layer, x.to(DEV).contiguous(), idx.to(DEV).contiguous(), w.to(DEV).contiguous(), ws, shared)
    y = ops.moe_prefill(*args)
    y2 = ops.moe_prefill(*args)
    torch.cuda.synchronize()
    assert ops.prefill_status(ws) == 0
    assert torch.equal(y, y2), "two calls must give identical bits"
    return y.cpu()


def test_olmoe_prefill_golden(golden_dir):
    g = np.load(golden_dir / "olmoe_prefill.npz")
    x = bits_to_bf16(g["x_bits"])
    idx, w = torch.from_numpy(g["idx"]), torch.from_numpy(g["w"])
    src = expert_source(SEED, 3, "olmoe", "q4_group128")
    experts = {int(e): src(int(e)) for e in set(idx.reshape(-1).tolist())}
    layer = stage_layer(experts, 64, 2048, 1024, "q4_group128", DEV)
    assert_parity(_run_prefill(layer, x, idx, w), bits_to_bf16(g["y_bits"]))


@pytest.mark.parametrize("layer_index", [0, 1, 2])
def test_qwen_prefill_golden(golden_dir, layer_index):
    from uma_qmoe_b200.ops import DeviceSharedExpert
    g = np.load(golden_dir / "qwen_layers.npz")
    enc = str(g[f"L{layer_index}_encoding"])
    src = expert_source(SEED, layer_index, "qwen", enc)
    x = bits_to_bf16(g["x8_bits"])
    idx = torch.from_numpy(g[f"L{layer_index}_i8"])
    w = torch.from_numpy(g[f"L{layer_index}_w8"])
    experts = {int(e): src(int(e)) for e in set(idx.reshape(-1).tolist())}
    layer = stage_layer(experts, 60, 2048, 1408, enc, DEV)
    assert_parity(_run_prefill(layer, x, idx, w), bits_to_bf16(g[f"L{layer_index}_y8_bits"]))
    sg, su, sd, sgate = (t.to(DEV).contiguous() for t in syn.shared_expert_weights(SEED, layer_index, syn.QWEN))
    b = _run_prefill(layer, x, idx, w, DeviceSharedExpert(sg, su, sd, sgate))
    assert_parity(b, bits_to_bf16(g[f"L{layer_index}_b8_bits"]))


def test_prefill_many_tokens_few_experts_matches_oracle():
    """300 tokens over 4 experts: several 128-route tiles per expert, ragged last tiles, one empty expert."""
    src = expert_source(SEED, 9, "olmoe", "q4_group128")
    tokens = 300
    rng = np.random.default_rng(5)
    idx = torch.from_numpy(np.stack([rng.permutation([0, 1, 2, 4, 5, 6, 7, 8])[:8] for _ in range(tokens)]).astype(np.int64))
    idx[:, 4:] = idx[:, :4]          # every token hits only 4 distinct experts, each twice
    w = torch.from_numpy(rng.random((tokens, 8), dtype=np.float32) / 8)
    used = sorted(set(idx.reshape(-1).tolist()))
    layer = stage_layer({e: src(e) for e in used}, 16, 2048, 1024, "q4_group128", DEV)
    x = syn.activations(SEED + 21, tokens)
    want = orc.moe_forward(x, idx, w, src, num_experts=64, top_k=8, qwen=False)
    assert_parity(_run_prefill(layer, x, idx, w), want)


@pytest.mark.parametrize("tokens", [500, 40, 5, 299])      # tensor-core kernel (ragged last CTA) / cluster kernel: ten
                                                            # clusters, two with a one-token tail, 75 with a ragged tail
@pytest.mark.parametrize("model,renorm", [("olmoe", True), ("olmoe", False), ("qwen", False)])
def test_router_matches_oracle(model, renorm, tokens):
    from uma_qmoe_b200 import ops
    shape = syn.OLMOE if model == "olmoe" else syn.QWEN
    wr = syn.router_weight(SEED, 1, shape, skew=1.5)
    x = syn.activations(SEED + 31, tokens)
    probs, w_ref, idx_ref = orc.router_topk(x, wr, shape.top_k, renorm)
    w, idx, logits = ops.route_topk(x.to(DEV), wr.to(DEV), shape.top_k, renorm, return_logits=True)
    w, idx, logits = w.cpu(), idx.cpu(), logits.cpu()
    ref_logits = torch.nn.functional.linear(x, wr)
    same_logits = (logits == ref_logits).all(dim=1)
    # BF16 logits are coarse, so equal probabilities are common.  Rows whose logits agree with the
    # oracle's and whose k-th and (k+1)-th probabilities differ must select the same expert SET with
    # the same weights; if no two of the top k+1 are equal the order must match too.
    srt = probs.sort(dim=1, descending=True).values
    k = shape.top_k
    boundary_clear = same_logits & (srt[:, k - 1] != srt[:, k])
    all_clear = same_logits & (srt[:, : k + 1].diff(dim=1) != 0).all(dim=1)
    # the kernel rounds an exactly summed dot product; the CPU GEMM of the oracle is off by one BF16 ulp on
    # about 1 logit in 5000, i.e. on 1-2 % of the rows
    if tokens >= 40:                                   # (with a handful of rows these shares are not statistics)
        assert same_logits.float().mean() >= 0.95 and boundary_clear.float().mean() > 0.85 and all_clear.any()
    assert torch.equal(idx[boundary_clear].sort(dim=1).values, idx_ref[boundary_clear].sort(dim=1).values)
    assert torch.allclose(w[boundary_clear].sort(dim=1).values, w_ref[boundary_clear].sort(dim=1).values,
                          rtol=2e-5, atol=1e-8)
    assert torch.equal(idx[all_clear], idx_ref[all_clear])
    assert torch.allclose(w[all_clear], w_ref[all_clear], rtol=2e-5, atol=1e-8)
    # every other row must still pick a valid top-k of its own logits
    own = torch.softmax(logits.float(), dim=1)
    chosen = own.gather(1, idx)
    kth = own.sort(dim=1, descending=True).values[:, shape.top_k - 1]
    assert bool((chosen >= kth[:, None] - 1e-9).all())
    assert int((~same_logits).sum()) <= max(1, 0.05 * x.shape[0])


@pytest.mark.parametrize("tokens,top_k,experts,dtype", [(8192, 8, 64, torch.int64), (5000, 4, 60, torch.int32),
                                                        (3, 8, 64, torch.int64)])
def test_route_sort_is_the_stable_sort_by_expert(tokens, top_k, experts, dtype):
    """Single-CTA and many-CTA sorts both equal a stable argsort; the tile list covers every route once."""
    from uma_qmoe_b200 import ops
    gen = torch.Generator().manual_seed(SEED + tokens)
    popularity = 1.0 / torch.arange(1, experts + 1, dtype=torch.float64) ** 1.2
    idx = torch.multinomial(popularity.expand(tokens, experts), top_k, replacement=False, generator=gen).to(dtype)
    w = torch.rand((tokens, top_k), generator=gen, dtype=torch.float32)
    r = ops.route_sort(idx.to(DEV), w.to(DEV), experts)
    torch.cuda.synchronize()
    assert int(r.status.item()) == 0
    flat = idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=experts)
    assert torch.equal(r.sorted_route.cpu().long(), order)
    assert torch.equal(r.counts.cpu().long(), counts)
    assert torch.equal(r.offsets.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]))
    assert torch.equal(r.route_pos.cpu().long()[order], torch.arange(flat.numel()))
    assert torch.equal(r.sorted_weight.cpu(), w.reshape(-1)[order])
    tiles = int(r.num_tiles.item())
    table = r.tile_table.cpu().view(3, r.max_tiles)[:, :tiles]
    covered = torch.zeros(flat.numel(), dtype=torch.int32)
    for e, row0, rows in table.t().tolist():
        assert (flat[order[row0:row0 + rows]] == e).all()
        covered[row0:row0 + rows] += 1
    assert (covered == 1).all()


def _stagewise(layer, x, idx, w, variant):
    """Prefill assembled from the exported stages, with the grouped GEMM kernel chosen explicitly."""
    from uma_qmoe_b200 import ops
    quant = layer.encoding != "bf16_le"
    r = ops.route_sort(idx, w, layer.num_experts)
    xs = ops.gather_rows(x, r.sorted_route, idx.shape[1], permute=quant)
    inter = ops.grouped_gemm(layer, 0, xs, r, permute_out=quant, variant=variant)
    yw = ops.grouped_gemm(layer, 1, inter, r, route_weight=r.sorted_weight, variant=variant)
    y = ops.combine_routes(yw, idx, r.route_pos)
    torch.cuda.synchronize()
    assert int(r.status.item()) == 0
    return inter, y


@pytest.mark.parametrize("encoding", ["q4_group128", "q8_group128", "bf16_le"])
def test_pair_kernel_matches_single_cta_kernel_and_oracle(encoding):
    """The persistent CTA-pair GEMM (cta_group::2) against the one-CTA-per-tile GEMM and the oracle: 700 tokens
    over 5 experts give full 256-route tiles, ragged tiles above and below 128 routes, and enough (tile, column)
    items that every cluster walks several of them with both accumulators in use."""
    src = expert_source(SEED, 3, "olmoe", encoding)
    tokens = 700
    rng = np.random.default_rng(11)
    pool = np.array([0, 2, 3, 5, 9])
    prob = np.array([0.45, 0.3, 0.15, 0.07, 0.03])
    idx = torch.from_numpy(np.stack([rng.choice(pool, size=2, replace=False, p=prob) for _ in range(tokens)]).astype(np.int64))
    w = torch.from_numpy(rng.random((tokens, 2), dtype=np.float32) / 2)
    layer = stage_layer({int(e): src(int(e)) for e in pool}, 16, 2048, 1024, encoding, DEV)
    x = syn.activations(SEED + 33, tokens)
    args = (layer, x.to(DEV), idx.to(DEV), w.to(DEV))
    inter1, y1 = _stagewise(*args, variant=1)
    inter2, y2 = _stagewise(*args, variant=2)
    inter2b, y2b = _stagewise(*args, variant=2)
    assert torch.equal(y2, y2b) and torch.equal(inter2, inter2b), "two calls must give identical bits"
    assert_parity(y2.cpu(), y1.cpu(), max_abs=4e-3)
    mismatch = (inter1 != inter2).float().mean().item()
    assert mismatch < 1e-3, f"intermediates differ in {mismatch:.2%} of the elements"
    want = orc.moe_forward(x, idx, w, src, num_experts=64, top_k=2, qwen=False)
    assert_parity(y2.cpu(), want)


def test_large_batch_prefill_matches_the_pair_kernel_and_the_oracle():
    """4096 tokens x top-8 (32768 routes: every persistent CTA walks many tiles) through umaq_moe_prefill vs the
    stages run on the CTA-pair kernel; a sample of tokens is checked against the oracle."""
    src = expert_source(SEED, 5, "olmoe", "q4_group128")
    tokens, experts = 4096, 16
    gen = torch.Generator().manual_seed(SEED + 77)
    popularity = 1.0 / torch.arange(1, experts + 1, dtype=torch.float64) ** 1.1
    idx = torch.multinomial(popularity.expand(tokens, experts), 8, replacement=False, generator=gen)
    w = torch.rand((tokens, 8), generator=gen, dtype=torch.float32) / 8
    layer = stage_layer({e: src(e) for e in range(experts)}, experts, 2048, 1024, "q4_group128", DEV)
    x = syn.activations(SEED + 34, tokens)
    y = _run_prefill(layer, x, idx, w)
    _, y2 = _stagewise(layer, x.to(DEV), idx.to(DEV), w.to(DEV), variant=2)
    assert_parity(y, y2.cpu(), max_abs=4e-3)
    sample = torch.arange(0, tokens, 512)
    want = orc.moe_forward(x[sample], idx[sample], w[sample], src, num_experts=experts, top_k=8, qwen=False)
    assert_parity(y[sample], want)


@pytest.mark.parametrize("encoding", ["q4_group128", "q8_group128", "bf16_le"])
def test_gate_up_gemm_by_index_equals_the_gemm_on_gathered_rows(encoding):
    """The gate/up GEMM that fetches its activation rows itself (cp.async producers writing the swizzled tile) must
    give the bits of the same GEMM on a gathered copy: full, ragged and half tiles, and an expert without routes."""
    from uma_qmoe_b200 import ops
    src = expert_source(SEED, 7, "olmoe", encoding)
    tokens = 777
    rng = np.random.default_rng(12)
    pool = np.array([0, 1, 3, 4, 7, 8, 11])
    idx = torch.from_numpy(np.stack([rng.choice(pool, 2, replace=False, p=[.5, .2, .1, .1, .05, .03, .02]) for _ in range(tokens)]))
    w = torch.rand((tokens, 2), generator=torch.Generator().manual_seed(3)) / 2
    layer = stage_layer({int(e): src(int(e)) for e in pool}, 16, 2048, 1024, encoding, DEV)
    x = syn.activations(SEED + 36, tokens).to(DEV)
    quant = encoding != "bf16_le"
    r = ops.route_sort(idx.to(DEV), w.to(DEV), layer.num_experts)
    xs = ops.gather_rows(x, r.sorted_route, 2, permute=quant)
    want = ops.grouped_gemm(layer, 0, xs, r, permute_out=quant, variant=1)
    source = ops.gather_rows(x, None, 1, permute=True) if quant else x
    got = ops.grouped_gemm_by_index(layer, source, r, 2, permute_out=quant)
    again = ops.grouped_gemm_by_index(layer, source, r, 2, permute_out=quant)
    torch.cuda.synchronize()
    assert int(r.status.item()) == 0
    assert torch.equal(got, want) and torch.equal(got, again)


def test_bf16_large_batch_takes_the_pair_kernel_by_default_and_matches_the_one_cta_kernel():
    """BF16 layers on 16,384 routes or more run on the CTA-pair kernel unless the caller picks one; the whole
    operator must agree with the stages run explicitly on the one-CTA kernel and with the oracle on a sample."""
    src = expert_source(SEED, 6, "olmoe", "bf16_le")
    tokens, experts = 2048, 16
    gen = torch.Generator().manual_seed(SEED + 78)
    idx = torch.stack([torch.randperm(experts, generator=gen)[:8] for _ in range(tokens)])
    w = torch.rand((tokens, 8), generator=gen, dtype=torch.float32) / 8
    layer = stage_layer({e: src(e) for e in range(experts)}, experts, 2048, 1024, "bf16_le", DEV)
    x = syn.activations(SEED + 35, tokens)
    y = _run_prefill(layer, x, idx, w)                                        # 16,384 routes: variant 0 -> pairs
    _, y1 = _stagewise(layer, x.to(DEV), idx.to(DEV), w.to(DEV), variant=1)
    _, y2 = _stagewise(layer, x.to(DEV), idx.to(DEV), w.to(DEV), variant=2)
    assert torch.equal(y, y2.cpu())
    assert_parity(y, y1.cpu(), max_abs=4e-3)
    sample = torch.arange(0, tokens, 256)
    want = orc.moe_forward(x[sample], idx[sample], w[sample], src, num_experts=experts, top_k=8, qwen=False)
    assert_parity(y[sample], want)


def test_operator_edge_shapes_through_the_registered_backend():
    """The public operator on an empty batch, on one token (decode kernels) and on two tokens (prefill kernels):
    same pack, results consistent with each other."""
    from uma_qmoe_b200 import custom_op, native_backend
    from uma_qmoe_b200.packs import InMemoryPack, expert_tensor_name
    from uma_qmoe_b200.formats import encode
    pack = InMemoryPack({0: "q4_group128"})
    packed = {}                                      # 8 distinct experts, repeated to fill the layer's 64
    for e in range(8):
        for proj, m in zip(("gate_proj", "up_proj", "down_proj"), syn.expert_weights(SEED, 0, e, syn.OLMOE)):
            packed[e, proj] = encode(m, "q4_group128")
    for e in range(64):
        for proj in ("gate_proj", "up_proj", "down_proj"):
            pack.add_packed(expert_tensor_name(0, e, proj), packed[e % 8, proj])
    native_backend.install_mixed_target_backend()
    handle = custom_op.register_expert_pack(pack)
    try:
        x = syn.activations(SEED + 3, 2).to(DEV)
        idx = torch.tensor([[0, 1, 2, 3, 4, 5, 6, 7], [7, 6, 5, 4, 3, 2, 1, 0]], device=DEV)
        w = torch.full((2, 8), 0.125, device=DEV)
        both = torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, True)
        one = torch.ops.uma_qmoe.moe_forward(x[:1], idx[:1], w[:1], 0, handle, True)
        none = torch.ops.uma_qmoe.moe_forward(x[:0], idx[:0], w[:0], 0, handle, True)
        assert none.shape == (0, 2048) and none.dtype == torch.bfloat16
        assert_parity(one.cpu(), both[:1].cpu(), max_abs=4e-3)
        three_d = torch.ops.uma_qmoe.moe_forward(x.reshape(1, 2, 2048), idx, w, 0, handle, True)
        assert three_d.shape == (1, 2, 2048) and torch.equal(three_d.reshape(2, 2048), both)
        with pytest.raises(RuntimeError, match=r"requires \[tokens, 8\] routes"):
            torch.ops.uma_qmoe.moe_forward(x, idx[:, :4], w[:, :4], 0, handle, True)
        with pytest.raises(RuntimeError, match="layer_index must be in"):
            torch.ops.uma_qmoe.moe_forward(x, idx, w, 16, handle, True)
    finally:
        custom_op.unregister_expert_pack(handle)


def test_reference_validator_and_route_trace_prefill(golden_dir):
    """The reference validator's 32-token case and the 128-token prefill event of layer 0 of its frozen route
    trace (32 of 64 experts hit, 53 routes on the busiest, un-normalised weights), against the reference's CPU
    outputs."""
    g = np.load(golden_dir / "reference_cases.npz")
    src = expert_source(SEED, int(g["layer"]), "olmoe", "q4_group128")
    layer = stage_layer({int(e): src(int(e)) for e in g["hit"]}, 64, 2048, 1024, "q4_group128", DEV)
    idx = torch.from_numpy(g["val_idx"]).repeat(32, 1)
    w = bits_to_bf16(g["val_w_bits"]).float().repeat(32, 1)
    assert_parity(_run_prefill(layer, bits_to_bf16(g["val_x32_bits"]), idx, w), bits_to_bf16(g["val_y32_bits"]))
    y = _run_prefill(layer, bits_to_bf16(g["trace_prefill_x_bits"]), torch.from_numpy(g["trace_prefill_idx"]),
                     torch.from_numpy(g["trace_prefill_w"]))
    assert_parity(y, bits_to_bf16(g["trace_prefill_y_bits"]))


def test_baseline_prefill_512_tokens_skewed_router():
    """The 512-token prefill configuration exactly: all 64 experts staged, routes from the skewed seeded router
    through the router kernel (some experts get no token, the busiest at least three times the mean), result
    against the CPU oracle."""
    from uma_qmoe_b200 import ops
    shape = syn.OLMOE
    src = expert_source(SEED, 2, "olmoe", "q4_group128")
    layer = stage_layer({e: src(e) for e in range(64)}, 64, 2048, 1024, "q4_group128", DEV)
    x = syn.activations(SEED + 51, 512)
    wr = syn.router_weight(SEED, 2, shape, skew=1.5)
    w, idx = ops.route_topk(x.to(DEV), wr.to(DEV), shape.top_k, True)
    w, idx = w.cpu(), idx.cpu()
    counts = torch.bincount(idx.reshape(-1), minlength=64)
    assert int(counts.min()) == 0 and int(counts.max()) >= 3 * counts.float().mean(), counts.tolist()
    want = orc.moe_forward(x, idx, w, src, num_experts=64, top_k=8, qwen=False)
    assert_parity(_run_prefill(layer, x, idx, w), want)


def test_stack_shape_8192_tokens_sampled_rows():
    """The expert-parallel stack's shape (8192 tokens x 64 experts x top-8, layer 0 of the benchmark stack) on one
    GPU; 64 sampled token rows against the CPU oracle, which dequantises the staged bytes of the experts they hit."""
    from uma_qmoe_b200 import ops
    from uma_qmoe_b200.stack import random_layer
    shape = syn.OLMOE
    dev = torch.device(DEV)
    layer = random_layer(shape, "q4_group128", SEED, dev)
    x = syn.activations(SEED, 8192)
    wr = syn.router_weight(SEED, 0, shape, skew=1.0)
    w, idx = ops.route_topk(x.to(dev), wr.to(dev), shape.top_k, True)
    y = _run_prefill(layer, x, idx.cpu(), w.cpu())
    rows = torch.arange(0, 8192, 128)
    idx_s, w_s = idx.cpu()[rows], w.cpu()[rows]

    def staged(e: int):
        def take(t, s, n, k):
            per = n * k // 2
            data = t[e * per:(e + 1) * per].cpu().numpy()
            scales = s[e * (n * k // 128):(e + 1) * (n * k // 128)].cpu().numpy()
            return orc.EncodedMatrix("q4_group128", (n, k), data, scales)
        return (take(layer.gate, layer.gate_scales, 1024, 2048), take(layer.up, layer.up_scales, 1024, 2048),
                take(layer.down, layer.down_scales, 2048, 1024))
    cache = {}
    src = lambda e: cache.setdefault(e, staged(e))
    want = orc.moe_forward(x[rows], idx_s, w_s, src, num_experts=64, top_k=8, qwen=False)
    assert_parity(y[rows], want)
