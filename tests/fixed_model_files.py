"""Builds the files a fixed-model host loads, with random weights: a Hugging Face checkpoint directory that holds
only the dense tensors (the index still lists every routed-expert tensor, as a real checkpoint's does) and a
TargetPack with the routed experts, written by the reference's own writer.

    python tests/fixed_model_files.py OUT_DIR [--layers 2] [--vocab 4096] [--seed 7]

The model is Qwen1.5-MoE-A2.7B-shaped per layer (hidden 2048, 16 heads, 60 experts of 1408, top-4 without
renormalisation, shared expert 5632 with a sigmoid gate); depth and vocabulary are reduced so that the files stay
around 2 GB and a CPU run of the same model takes seconds.  Needs the reference package (``oracle/_ref``, made by
``oracle/make_ref.py``) for the pack writer; prints the paths and identities as one JSON line.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"
MODEL_ID, MODEL_REVISION = "Qwen/Qwen1.5-MoE-A2.7B", "1a758c50ecb6350748b9ce0a99d2352fd9fc11c9"
POLICY_ID = "synthetic-bf16-then-q8"


def qwen_config(layers: int, vocab: int):
    import transformers
    return transformers.Qwen2MoeConfig(vocab_size=vocab, hidden_size=2048, num_hidden_layers=layers,
                                       num_attention_heads=16, num_key_value_heads=16, max_position_embeddings=4096,
                                       intermediate_size=5632, moe_intermediate_size=1408,
                                       shared_expert_intermediate_size=5632, num_experts=60, num_experts_per_tok=4,
                                       norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[],
                                       initializer_range=0.05, tie_word_embeddings=False)


def layer_policy(layers: int) -> dict[int, str]:
    """The first two thirds of the layers BF16, the rest Q8 (the mixed policy of the reference's Qwen target),
    over the 24 layers a Qwen TargetPack policy must name."""
    table = {i: ("bf16_le" if i < max(1, layers * 2 // 3) else "q8_group128") for i in range(layers)}
    table.update({i: "q8_group128" for i in range(layers, 24)})
    return table


def build(out: Path, layers: int = 2, vocab: int = 4096, seed: int = 7) -> dict:
    import transformers
    from safetensors.torch import save_file
    if not (REF / "uma_qmoe" / "target_pack.py").exists():
        raise RuntimeError("the reference package is not installed under oracle/_ref (run oracle/make_ref.py)")
    sys.path.insert(0, str(REF))
    from uma_qmoe.target_pack import write_target_pack

    out.mkdir(parents=True, exist_ok=True)
    model_dir, pack = out / "model", out / "experts.uqmotpk"
    model_dir.mkdir(exist_ok=True)
    config = qwen_config(layers, vocab)
    torch.manual_seed(seed)
    model = transformers.Qwen2MoeForCausalLM(config).to(torch.bfloat16).eval()
    state = model.state_dict()
    dense = {k: v.contiguous() for k, v in state.items() if ".mlp.experts." not in k}
    config.save_pretrained(model_dir)
    shard = "model-00001-of-00001.safetensors"
    save_file(dense, str(model_dir / shard), metadata={"format": "pt"})
    inter = config.moe_intermediate_size

    def expert_tensors():
        for l in range(layers):
            gate_up = state[f"model.layers.{l}.mlp.experts.gate_up_proj"]        # [E, 2I, H]
            down = state[f"model.layers.{l}.mlp.experts.down_proj"]              # [E, H, I]
            for e in range(config.num_experts):
                yield f"model.layers.{l}.mlp.experts.{e}.gate_proj.weight", gate_up[e, :inter].float().numpy()
                yield f"model.layers.{l}.mlp.experts.{e}.up_proj.weight", gate_up[e, inter:].float().numpy()
                yield f"model.layers.{l}.mlp.experts.{e}.down_proj.weight", down[e].float().numpy()

    weight_map = {name: shard for name in dense}
    for l in range(layers):
        for e in range(config.num_experts):
            for p in ("gate_proj", "up_proj", "down_proj"):
                weight_map[f"model.layers.{l}.mlp.experts.{e}.{p}.weight"] = "experts-are-in-the-pack.safetensors"
    (model_dir / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    manifest = hashlib.sha256(json.dumps(sorted(weight_map.items())).encode()).hexdigest()
    if pack.exists():
        pack.unlink()
    write_target_pack(pack, expert_tensors(), model_id=MODEL_ID, model_revision=MODEL_REVISION,
                      model_manifest_sha256=manifest, policy_id=POLICY_ID, layer_encodings=layer_policy(layers),
                      policy_evidence_sha256=hashlib.sha256(b"synthetic policy").hexdigest())
    return {"model_directory": str(model_dir), "pack": str(pack), "model_manifest_sha256": manifest,
            "policy_id": POLICY_ID, "layers": layers, "vocab": vocab, "seed": seed}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("out", type=Path)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=7)
    args = ap.parse_args()
    print(json.dumps(build(args.out, args.layers, args.vocab, args.seed)))


if __name__ == "__main__":
    main()
