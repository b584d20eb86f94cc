"""Generate the golden fixtures in this directory by running the UMA-QMoE reference itself.

Run once, in a container that has the reference checked out (it cannot travel
to the GPU machines, the ``.npz`` files do):

    python tests/golden/make_golden.py --reference /path/to/reference

For every case the script builds seeded synthetic weights
(``uma_qmoe_b200.synthetic``), writes them into a real ExpertPack / TargetPack
with the reference's own writers (i.e. its own quantiser), runs the
reference's CPU correctness dispatch ``torch.ops.uma_qmoe.moe_forward`` /
``qwen_moe_forward`` (``performance_mode=False``), the Hugging Face router and,
for Qwen, the reference's ``QuantizedQwenMoEBlock`` -- and stores inputs,
outputs and SHA-256 digests of the packed bytes.  Weights are not stored (they
are regenerated from the seed); their digests are.
"""

from __future__ import annotations

import argparse
import hashlib
import sys
import tempfile
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from uma_qmoe_b200 import synthetic as syn  # noqa: E402

SEED = 20260917
REV = "0" * 40
SHA = "0" * 64


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).numpy().astype(np.uint16)


def digest(*chunks: bytes) -> str:
    h = hashlib.sha256()
    for c in chunks:
        h.update(c)
    return h.hexdigest()


def name_of(layer: int, expert: int, proj: str) -> str:
    return f"model.layers.{layer}.mlp.experts.{expert}.{proj}_proj.weight"


def expert_stream(seed: int, layer: int, experts: list[int], shape: syn.ModelShape):
    for e in experts:
        g, u, d = syn.expert_weights(seed, layer, e, shape)
        yield name_of(layer, e, "gate"), g
        yield name_of(layer, e, "up"), u
        yield name_of(layer, e, "down"), d


def pack_digests(reader, layer: int, experts: list[int]) -> dict[str, str]:
    out = {}
    for e in experts:
        for p in ("gate", "up", "down"):
            data, scales, _meta = reader.tensor_views(name_of(layer, e, p))
            out[f"sha_{e}_{p}"] = digest(bytes(data), bytes(scales))
            data.release(); scales.release()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "src"))
    from transformers.models.olmoe.modeling_olmoe import OlmoeTopKRouter
    from transformers.models.qwen2_moe.modeling_qwen2_moe import Qwen2MoeMLP, Qwen2MoeTopKRouter
    from uma_qmoe import custom_op as ref_op
    from uma_qmoe.expert_pack import ExpertPackReader, write_expert_pack
    from uma_qmoe.q4 import quantize_q4
    from uma_qmoe.qwen_compressed_loader import QuantizedQwenMoEBlock
    from uma_qmoe.target_pack import TargetPackReader, encode_target_tensor, write_target_pack

    ref_op.register_moe_forward()
    torch.manual_seed(0)
    tmp = Path(tempfile.mkdtemp(prefix="umaq_golden_"))
    meta = {"torch": torch.__version__, "numpy": np.__version__}
    import transformers
    meta["transformers"] = transformers.__version__

    # ---- codec vectors on odd sizes (tail group, odd nibble count) -------------
    codec = {}
    for i, n in enumerate((1, 129, 255, 1000)):
        v = syn.normal_bf16((SEED, 7, i), (n,), 0.02)
        if i == 2:
            v[:128] = 0.0                       # an all-zero group -> scale 1.0
        q4 = quantize_q4(v)
        q8 = encode_target_tensor(v, "q8_group128")
        b16 = encode_target_tensor(v, "bf16_le")
        codec[f"in_{i}"] = v
        codec[f"q4_packed_{i}"] = np.frombuffer(q4.packed, np.uint8)
        codec[f"q4_scales_{i}"] = np.frombuffer(q4.scales, "<f4")
        codec[f"q8_data_{i}"] = np.frombuffer(q8.data, np.int8)
        codec[f"q8_scales_{i}"] = np.frombuffer(q8.scales, "<f4")
        codec[f"bf16_{i}"] = np.frombuffer(b16.data, "<u2")
    np.savez_compressed(HERE / "codec.npz", **codec)

    # ---- OLMoE: HF router + operator, 1 token (config-0 style) ----------------
    shape = syn.OLMOE
    cfg = types.SimpleNamespace(num_experts_per_tok=8, num_experts=64, norm_topk_prob=True,
                                hidden_size=2048)
    router = OlmoeTopKRouter(cfg).to(torch.bfloat16)
    wr = syn.router_weight(SEED, 0, shape)
    with torch.no_grad():
        router.weight.copy_(wr)
    x1 = syn.activations(SEED + 1, 1)
    with torch.no_grad():
        probs, w_norm, idx = router(x1)
        router.norm_topk_prob = False
        _p, w_raw, idx2 = router(x1)
    assert torch.equal(idx, idx2)
    hit = sorted(set(idx.reshape(-1).tolist()))
    pack_path = tmp / "olmoe_decode.uqmoepk"
    write_expert_pack(pack_path, expert_stream(SEED, 0, hit, shape), model_id="allenai/OLMoE-1B-7B-0125",
                      model_revision=REV, model_manifest_sha256=SHA)
    reader = ExpertPackReader(pack_path)
    handle = ref_op.register_expert_pack(reader)
    y_norm = torch.ops.uma_qmoe.moe_forward(x1, idx, w_norm, 0, handle, False)
    y_raw = torch.ops.uma_qmoe.moe_forward(x1, idx, w_raw, 0, handle, False)
    np.savez_compressed(
        HERE / "olmoe_decode.npz", seed=SEED, x_bits=bits(x1), probs=probs.numpy(),
        w_norm=w_norm.numpy(), w_raw=w_raw.numpy(), idx=idx.numpy(),
        y_norm_bits=bits(y_norm), y_raw_bits=bits(y_raw), router_sha=digest(bits(wr).tobytes()),
        meta=str(meta), **pack_digests(reader, 0, hit))
    ref_op.unregister_expert_pack(handle)
    reader.close()

    # ---- OLMoE: 24-token prefill, skewed routes over 12 experts, layer 3 -------
    tokens, pool = 24, 12
    xp = syn.activations(SEED + 2, tokens)
    idx_p, w_p = syn.skewed_routes(SEED + 2, tokens, shape, pool)
    idx_p[5, 1] = idx_p[5, 0]                      # one token routes twice to one expert
    hit = sorted(set(idx_p.reshape(-1).tolist()))
    pack_path = tmp / "olmoe_prefill.uqmoepk"
    write_expert_pack(pack_path, expert_stream(SEED, 3, hit, shape), model_id="allenai/OLMoE-1B-7B-0125",
                      model_revision=REV, model_manifest_sha256=SHA)
    reader = ExpertPackReader(pack_path)
    handle = ref_op.register_expert_pack(reader)
    y_p = torch.ops.uma_qmoe.moe_forward(xp.reshape(2, 12, 2048), idx_p, w_p, 3, handle, False)
    np.savez_compressed(HERE / "olmoe_prefill.npz", seed=SEED, layer=3, x_bits=bits(xp),
                        idx=idx_p.numpy(), w=w_p.numpy(), y_bits=bits(y_p.reshape(tokens, 2048)),
                        **pack_digests(reader, 3, hit))
    ref_op.unregister_expert_pack(handle)
    reader.close()

    # ---- Qwen: TargetPack with one layer of each encoding ----------------------
    shape = syn.QWEN
    qcfg = types.SimpleNamespace(num_experts_per_tok=4, num_experts=60, norm_topk_prob=False,
                                 hidden_size=2048, intermediate_size=5632, hidden_act="silu")
    qrouter = Qwen2MoeTopKRouter(qcfg).to(torch.bfloat16)
    shared = Qwen2MoeMLP(qcfg, intermediate_size=5632).to(torch.bfloat16)
    shared_gate = torch.nn.Linear(2048, 1, bias=False).to(torch.bfloat16)
    encodings = {0: "bf16_le", 1: "q8_group128", 2: "q4_group128"}
    policy = {i: encodings.get(i, "q4_group128") for i in range(24)}
    x1 = syn.activations(SEED + 3, 1)
    x8 = syn.activations(SEED + 4, 8)
    routes = {}
    tensors = []
    for layer in encodings:
        wr = syn.router_weight(SEED, layer, shape)
        with torch.no_grad():
            qrouter.weight.copy_(wr)
            r1 = qrouter(x1)
            r8 = qrouter(x8)
        routes[layer] = (r1, r8)
        hit = sorted(set(r1[2].reshape(-1).tolist()) | set(r8[2].reshape(-1).tolist()))
        tensors.append((layer, hit))
    pack_path = tmp / "qwen.uqmotpk"

    def qwen_stream():
        for layer, hit in tensors:
            yield from expert_stream(SEED, layer, hit, shape)

    write_target_pack(pack_path, qwen_stream(), model_id="Qwen/Qwen1.5-MoE-A2.7B", model_revision=REV,
                      model_manifest_sha256=SHA, policy_id="golden_mixed", layer_encodings=policy,
                      policy_evidence_sha256=SHA)
    reader = TargetPackReader(pack_path)
    handle = ref_op.register_target_pack(reader)
    out = {"seed": SEED, "x1_bits": bits(x1), "x8_bits": bits(x8)}
    for layer, hit in tensors:
        (p1, w1, i1), (p8, w8, i8) = routes[layer]
        y1 = torch.ops.uma_qmoe.qwen_moe_forward(x1, i1, w1, layer, handle, False)
        y8 = torch.ops.uma_qmoe.qwen_moe_forward(x8, i8, w8, layer, handle, False)
        sg, su, sd, sgate = syn.shared_expert_weights(SEED, layer, shape)
        with torch.no_grad():
            shared.gate_proj.weight.copy_(sg); shared.up_proj.weight.copy_(su)
            shared.down_proj.weight.copy_(sd); shared_gate.weight.copy_(sgate)
            qrouter.weight.copy_(syn.router_weight(SEED, layer, shape))
            block = QuantizedQwenMoEBlock(qrouter, shared, shared_gate, layer_index=layer,
                                          pack_handle=handle, performance_mode=False)
            b1 = block(x1.reshape(1, 1, 2048))
            b8 = block(x8.reshape(1, 8, 2048))
        out.update({f"L{layer}_w1": w1.numpy(), f"L{layer}_i1": i1.numpy(), f"L{layer}_w8": w8.numpy(),
                    f"L{layer}_i8": i8.numpy(), f"L{layer}_y1_bits": bits(y1), f"L{layer}_y8_bits": bits(y8),
                    f"L{layer}_b1_bits": bits(b1.reshape(1, 2048)), f"L{layer}_b8_bits": bits(b8.reshape(8, 2048)),
                    f"L{layer}_encoding": policy[layer]})
        out.update({f"L{layer}_{k}": v for k, v in pack_digests(reader, layer, hit).items()})
    np.savez_compressed(HERE / "qwen_layers.npz", **out)
    ref_op.unregister_expert_pack(handle)
    reader.close()

    # ---- a tiny pack file of each container format, for the pack readers -------
    small = [(name_of(0, e, p), syn.normal_bf16((SEED, 9, e, i), s, 0.02))
             for e in range(2) for i, (p, s) in enumerate((("gate", (4, 256)), ("up", (4, 256)), ("down", (256, 4))))]
    p1 = HERE / "tiny.uqmoepk"
    p2 = HERE / "tiny.uqmotpk"
    for p in (p1, p2):
        p.unlink(missing_ok=True)
    write_expert_pack(p1, small, model_id="allenai/OLMoE-1B-7B-0125", model_revision=REV,
                      model_manifest_sha256=SHA)
    small_t = small + [(name_of(1, e, p), v) for (n, v), (e, p) in
                       zip(small, [(e, p) for e in range(2) for p in ("gate", "up", "down")])]
    small_t += [(name_of(2, e, p), v) for (n, v), (e, p) in
                zip(small, [(e, p) for e in range(2) for p in ("gate", "up", "down")])]
    write_target_pack(p2, small_t, model_id="allenai/OLMoE-1B-7B-0125", model_revision=REV,
                      model_manifest_sha256=SHA, policy_id="tiny",
                      layer_encodings={i: ("q4_group128", "q8_group128", "bf16_le")[i % 3] for i in range(16)},
                      policy_evidence_sha256=SHA)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
