"""The kernels inside a Hugging Face model: a two-layer model with the real MoE layer shapes (Qwen1.5-MoE-A2.7B:
60 experts, top-4, intermediate 1408, shared expert 5632; OLMoE: 64 experts, top-8, intermediate 1024), random
weights, its sparse blocks swapped for this package's blocks.  With ``bf16_le`` experts the weights are the same
numbers, so the logits must agree with the unmodified model to BF16 accumulation noise, in prefill and in
single-token decode steps; quantised experts must stay close to that."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tiny(kind: str):
    import transformers
    common = dict(vocab_size=1024, hidden_size=2048, num_hidden_layers=2, num_attention_heads=16,
                  num_key_value_heads=16, max_position_embeddings=256, intermediate_size=1024)
    if kind == "qwen":
        cfg = transformers.Qwen2MoeConfig(moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
                                          num_experts=60, num_experts_per_tok=4, norm_topk_prob=False,
                                          decoder_sparse_step=1, mlp_only_layers=[], **common)
        cls = transformers.Qwen2MoeForCausalLM
    else:
        cfg = transformers.OlmoeConfig(num_experts=64, num_experts_per_tok=8, norm_topk_prob=False, **common)
        cls = transformers.OlmoeForCausalLM
    torch.manual_seed(1234)
    with torch.device(DEV):
        model = cls(cfg).to(torch.bfloat16).eval()
    # the default initialisation gives a router that is almost uniform: spread the logits so that top-k is decisive
    with torch.no_grad():
        for layer in model.model.layers:
            layer.mlp.gate.weight.mul_(20.0)
    return model


@pytest.mark.parametrize("kind", ["qwen", "olmoe"])
def test_swapped_blocks_reproduce_the_model(kind):
    from uma_qmoe_b200.host import greedy_decode, install_quantized_blocks
    model = _tiny(kind)
    prompt = torch.randint(0, 1024, (1, 24), generator=torch.Generator().manual_seed(7)).to(DEV)
    want = greedy_decode(model, prompt, 5)                       # unmodified HF model: prefill + 4 decode steps
    with install_quantized_blocks(model, "bf16_le") as host:
        assert host.evidence["sparse_layers"] == 2 and host.evidence["dequantized_weight_bytes"] == 0
        assert not hasattr(model.model.layers[0].mlp, "experts")
        got = greedy_decode(model, prompt[:, :24], 1)           # same prompt: logits of the prefill
        # BF16 accumulation noise plus, now and then, a different k-th expert where two router probabilities are
        # one BF16 step apart (the logits here are about 3 in magnitude)
        scale = want["logits"][0].abs().max().item()
        bound = 0.04 * scale + 4e-2
        assert (got["logits"][0] - want["logits"][0]).abs().max().item() <= bound
        # teacher-forced decode steps: feed the reference's tokens so that both runs see the same inputs
        forced = torch.cat([prompt, torch.tensor([want["tokens"][:4]], device=DEV)], dim=1)
        with torch.no_grad():
            out = model(input_ids=prompt, use_cache=True)
            cache = out.past_key_values
            for step in range(4):
                out = model(input_ids=forced[:, 24 + step:25 + step], past_key_values=cache, use_cache=True)
                cache = out.past_key_values
                diff = (out.logits[0, -1].float().cpu() - want["logits"][step + 1]).abs().max().item()
                assert diff <= bound, (step, diff)


def test_quantised_policy_stays_close_to_the_bf16_model():
    from uma_qmoe_b200.host import greedy_decode, install_quantized_blocks
    prompt = torch.randint(0, 1024, (1, 16), generator=torch.Generator().manual_seed(8)).to(DEV)
    ref = _tiny("qwen")
    want = greedy_decode(ref, prompt, 1)["logits"][0]
    del ref
    torch.cuda.empty_cache()
    model = _tiny("qwen")                                        # same seed: the same weights
    with install_quantized_blocks(model, {0: "q8_group128", 1: "q4_group128"}) as host:
        assert host.layer_encodings == {0: "q8_group128", 1: "q4_group128"}
        got = greedy_decode(model, prompt, 3)
        cos = torch.nn.functional.cosine_similarity(got["logits"][0], want, dim=0).item()
        assert cos > 0.98, cos
        assert len(got["tokens"]) == 3 and len(got["tpot_ms"]) == 2 and got["ttft_ms"] > 0


def test_graphed_decode_equals_the_eager_loop():
    """The decode step captured in a CUDA graph (static cache, arg-max and position update on the device) must
    generate the tokens of the eager loop, twice in a row with the same decoder."""
    from uma_qmoe_b200.host import greedy_decode, greedy_decode_graphed, install_quantized_blocks
    model = _tiny("qwen")
    prompt = torch.randint(0, 1024, (1, 20), generator=torch.Generator().manual_seed(9)).to(DEV)
    with install_quantized_blocks(model, {0: "q8_group128", 1: "bf16_le"}):
        eager = greedy_decode(model, prompt, 8)
        first = greedy_decode_graphed(model, prompt, 8, keep_logits=True)
        again = greedy_decode_graphed(model, prompt, 8, decoder=first["decoder"])
        assert first["tokens"] == again["tokens"]
        scale = eager["logits"].abs().max().item()
        assert (first["logits"] - eager["logits"]).abs().max().item() <= 0.04 * scale + 4e-2
        margin = eager["logits"].topk(2, dim=-1).values
        decisive = (margin[:, 0] - margin[:, 1]) > 0.1 * scale          # steps whose arg-max is not a near-tie
        prefix = 0
        while prefix < 8 and eager["tokens"][prefix] == first["tokens"][prefix]:
            prefix += 1
        assert prefix == 8 or not bool(decisive[prefix]), (prefix, eager["tokens"], first["tokens"])
