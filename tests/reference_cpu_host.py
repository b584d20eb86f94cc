"""CPU correctness host built from the reference package itself: the Hugging Face model on CPU with every ``mlp``
replaced by the reference's ``QuantizedQwenMoEBlock`` (``performance_mode=False``, i.e. its CPU path behind
``torch.ops.uma_qmoe.qwen_moe_forward``) reading the pack through the reference's ``TargetPackReader``.

    python tests/reference_cpu_host.py FILES_JSON PROMPT_IDS NEW_TOKENS

FILES_JSON is the line ``tests/fixed_model_files.py`` printed.  The reference's own ``load_fixed_qwen`` cannot be
called on a reduced-depth checkpoint (it insists on 24 layers and 4320 skipped tensors), so this script does its
steps with the reference's classes: reader, operator registration, block swap, dense tensors by name.  Runs in a
process of its own because the reference and the package under test define the same ``torch.library`` namespace.
Prints one JSON line: the generated ids and, per generated position, the two largest logits and their ids.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "oracle" / "_ref"))


def main() -> None:
    files = json.loads(sys.argv[1])
    prompt = [int(t) for t in sys.argv[2].split(",")]
    new_tokens = int(sys.argv[3])
    from safetensors import safe_open
    from transformers import AutoConfig, AutoModelForCausalLM
    from uma_qmoe.custom_op import register_expert_pack, register_moe_forward, unregister_expert_pack
    from uma_qmoe.qwen_compressed_loader import QuantizedQwenMoEBlock
    from uma_qmoe.target_pack import TargetPackReader

    root = Path(files["model_directory"])
    config = AutoConfig.from_pretrained(root, local_files_only=True)
    reader = TargetPackReader(files["pack"], expected_model_id="Qwen/Qwen1.5-MoE-A2.7B",
                              expected_model_manifest_sha256=files["model_manifest_sha256"],
                              expected_policy_id=files["policy_id"])
    register_moe_forward()
    handle = register_expert_pack(reader)
    try:
        torch.manual_seed(0)
        model = AutoModelForCausalLM.from_config(config, dtype=torch.bfloat16)
        for index, layer in enumerate(model.model.layers):
            old = layer.mlp
            layer.mlp = QuantizedQwenMoEBlock(old.gate, old.shared_expert, old.shared_expert_gate, layer_index=index,
                                              pack_handle=handle, performance_mode=False)
        weight_map = json.loads((root / "model.safetensors.index.json").read_text())["weight_map"]
        wanted = set(model.state_dict())
        loaded = set()
        with torch.no_grad():
            for shard in sorted({s for n, s in weight_map.items() if n in wanted}):
                with safe_open(root / shard, framework="pt", device="cpu") as source:
                    for name in source.keys():
                        if name in wanted:
                            model.get_parameter(name).copy_(source.get_tensor(name))
                            loaded.add(name)
        assert loaded == wanted, sorted(wanted - loaded)[:4]
        model.eval()
        ids = torch.tensor([prompt])
        tokens, top2 = [], []
        with torch.no_grad():
            out = model(input_ids=ids, use_cache=True)
            for step in range(new_tokens):
                logits = out.logits[0, -1].float()
                best = torch.topk(logits, 2)
                tokens.append(int(best.indices[0]))
                top2.append([int(best.indices[0]), float(best.values[0]), int(best.indices[1]), float(best.values[1])])
                if step + 1 < new_tokens:
                    out = model(input_ids=torch.tensor([[tokens[-1]]]), past_key_values=out.past_key_values, use_cache=True)
        # the full last-position logits of the prefill, for a direct comparison
        print(json.dumps({"tokens": tokens, "top2": top2}))
    finally:
        unregister_expert_pack(handle)
        reader.close()


if __name__ == "__main__":
    main()
