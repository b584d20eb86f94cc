"""A fixed-model host loaded from files (checkpoint directory + TargetPack) the way the reference's
``load_fixed_qwen`` does it, against a CPU host built from the reference package on the same files."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
PROMPT = [11, 222, 3333, 444, 55, 666, 777, 888]
NEW_TOKENS = 2


def _last_json(text: str) -> dict:
    lines = [t for t in text.splitlines() if t.startswith("{")]
    assert lines, text[-2000:]
    return json.loads(lines[-1])


@pytest.mark.gpu
def test_fixed_qwen_host_from_files_generates_the_reference_cpu_hosts_tokens(tmp_path):
    """Two layers of the Qwen1.5-MoE layer shape (layer 0 BF16 experts, layer 1 Q8, shared experts, 60 experts top-4),
    dense tensors from Safetensors, experts from a TargetPack the reference's writer made.  Greedy ids for an 8-token
    prompt + 2 generated tokens must equal those of the reference package running the same files on CPU
    (``performance_mode=False``); where they differ, the CPU host's logit margin at the first difference must be
    within BF16 noise, and is reported."""
    if not (ROOT / "oracle" / "_ref" / "uma_qmoe" / "target_pack.py").exists():
        pytest.skip("the reference package is not installed under oracle/_ref")
    made = subprocess.run([sys.executable, str(ROOT / "tests" / "fixed_model_files.py"), str(tmp_path), "--layers", "2"],
                          capture_output=True, text=True, timeout=1200)
    assert made.returncode == 0, made.stderr[-2000:]
    files = _last_json(made.stdout)
    cpu = subprocess.Popen([sys.executable, str(ROOT / "tests" / "reference_cpu_host.py"), json.dumps(files),
                            ",".join(map(str, PROMPT)), str(NEW_TOKENS)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        from uma_qmoe_b200.fixed_loader import load_fixed_qwen
        with load_fixed_qwen(files["model_directory"], files["pack"], model_manifest_sha256=files["model_manifest_sha256"],
                             device="cuda:0", performance_mode=True, target_policy_id=files["policy_id"],
                             expected_layers=2) as host:
            ev = host.evidence
            assert ev["quantized_moe_block_count"] == 2 and ev["skipped_expert_tensor_count"] == 2 * 60 * 3
            assert ev["expert_parameter_count"] == 0 and ev["expert_pack_mapping_count"] == 1
            assert host.expert_pack.layer_encoding(0) == "bf16_le" and host.expert_pack.layer_encoding(1) == "q8_group128"
            ids = torch.tensor([PROMPT], device="cuda:0")
            tokens, logits = [], []
            with torch.no_grad():
                out = host.model(input_ids=ids, use_cache=True)                    # prefill kernels (8 tokens)
                for step in range(NEW_TOKENS):
                    row = out.logits[0, -1].float()
                    logits.append(row.cpu())
                    tokens.append(int(row.argmax()))
                    if step + 1 < NEW_TOKENS:                                       # decode kernels (1 token)
                        out = host.model(input_ids=torch.tensor([[tokens[-1]]], device="cuda:0"),
                                         past_key_values=out.past_key_values, use_cache=True)
            host.model.model.layers[0].mlp                                          # still a block of this package
        stdout, stderr = cpu.communicate(timeout=1200)
    finally:
        if cpu.poll() is None:
            cpu.kill()
    assert cpu.returncode == 0, stderr[-2000:]
    want = _last_json(stdout)
    for step, (tid, top) in enumerate(zip(tokens, want["top2"])):
        cpu_id, cpu_best = top[0], top[1]
        # the same position's logits on the device agree with the CPU host's two largest
        assert abs(float(logits[step][cpu_id]) - cpu_best) <= 0.25, (step, float(logits[step][cpu_id]), cpu_best)
        if tid != cpu_id:
            margin = cpu_best - (top[3] if tid == top[2] else float("-inf"))
            assert margin <= 0.125, f"ids differ at generated position {step}: {tid} vs {cpu_id}, CPU margin {margin}"
            break                                                                   # later positions saw different inputs
    print(json.dumps({"device_tokens": tokens, "cpu_tokens": want["tokens"], "cpu_top2": want["top2"]}))


def test_fixed_loader_refuses_what_the_reference_refuses(tmp_path):
    """The checks that come before any device work: architecture, pack kind against policy id, model identity."""
    import transformers

    from tests.fixed_model_files import qwen_config
    from uma_qmoe_b200.fixed_loader import load_fixed_olmoe, load_fixed_qwen
    from uma_qmoe_b200.formats import ContractError
    golden = ROOT / "tests" / "golden"
    wrong = tmp_path / "three_layers"
    qwen_config(3, 512).save_pretrained(wrong)
    with pytest.raises(ContractError, match="unexpected fixed Qwen architecture"):
        load_fixed_qwen(wrong, golden / "tiny.uqmotpk", model_manifest_sha256="0" * 64, target_policy_id="tiny")
    ok = tmp_path / "qwen"
    qwen_config(24, 512).save_pretrained(ok)
    with pytest.raises(ContractError, match="requires a policy id"):
        load_fixed_qwen(ok, golden / "tiny.uqmotpk", model_manifest_sha256="0" * 64)
    with pytest.raises(ContractError, match="cannot satisfy a TargetPack policy id"):
        load_fixed_qwen(ok, golden / "tiny.uqmoepk", model_manifest_sha256="0" * 64, target_policy_id="tiny")
    with pytest.raises(ContractError, match="model id mismatch"):          # the tiny packs name the OLMoE model
        load_fixed_qwen(ok, golden / "tiny.uqmotpk", model_manifest_sha256="0" * 64, target_policy_id="tiny")
    olmoe = tmp_path / "olmoe"
    transformers.OlmoeConfig(vocab_size=512, hidden_size=2048, intermediate_size=1024, num_hidden_layers=16,
                             num_attention_heads=16, num_experts=64, num_experts_per_tok=8).save_pretrained(olmoe)
    with pytest.raises(ContractError, match="model revision mismatch"):
        load_fixed_olmoe(olmoe, golden / "tiny.uqmoepk", model_manifest_sha256="0" * 64)
    with pytest.raises(ContractError, match="cannot read compressed OLMoE pack"):
        load_fixed_olmoe(olmoe, tmp_path / "missing.uqmoepk", model_manifest_sha256="0" * 64)
