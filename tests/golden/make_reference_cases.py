"""Golden vectors for the reference's own validation inputs, made by running the reference itself.

    python tests/golden/make_reference_cases.py --reference /path/to/reference

Writes ``reference_cases.npz`` beside this script:

* the inputs of the reference's GPU validator (``benchmarks/runners/validate_packed_q4_kernel.py:151-178``:
  hidden = linspace(-0.5, 0.5) in BF16, experts 0..7, routing weights 0.125 in BF16; one token, and 32 tokens
  with the same routes) and what the reference's CPU correctness dispatch returns for them;
* one layer of the reference's frozen route trace
  (``benchmarks/traces/olmoe_1b_7b_0125_128x32_greedy_v1.json`` read through
  ``uma_qmoe.route_trace.iter_replay_events``, ``src/uma_qmoe/route_trace.py:382-404``): the 128-token prefill
  event and the first decode event of layer 0 -- real, un-normalised top-8 routes with realistic skew -- and
  the CPU correctness output for seeded activations.

Expert weights are the seeded synthetic ones of layer 0 (``uma_qmoe_b200.synthetic``), packed by the
reference's own writer; they are regenerated from the seed by the tests, not stored.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from uma_qmoe_b200 import synthetic as syn  # noqa: E402

SEED = 20260917
LAYER = 0


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).numpy().astype(np.uint16)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    ref = Path(args.reference)
    sys.path.insert(0, str(ref / "src"))
    from uma_qmoe import custom_op as ref_op
    from uma_qmoe.expert_pack import ExpertPackReader, write_expert_pack
    from uma_qmoe.route_trace import iter_replay_events

    trace = json.loads((ref / "benchmarks" / "traces" / "olmoe_1b_7b_0125_128x32_greedy_v1.json").read_text())
    events = [e for e in iter_replay_events(trace) if e["layer_index"] == LAYER]
    prefill = next(e for e in events if e["phase"] == "prefill")
    decode = next(e for e in events if e["phase"] == "decode")

    def routes(event):
        n = event["token_count"]
        idx = torch.tensor(event["expert_indices"], dtype=torch.int64).reshape(n, 8)
        w = torch.tensor(event["routing_weights"], dtype=torch.float32).reshape(n, 8)
        return idx, w

    p_idx, p_w = routes(prefill)
    d_idx, d_w = routes(decode)
    hit = sorted(set(range(8)) | set(p_idx.reshape(-1).tolist()) | set(d_idx.reshape(-1).tolist()))
    shape = syn.OLMOE

    def stream():
        for e in hit:
            for proj, m in zip(("gate", "up", "down"), syn.expert_weights(SEED, LAYER, e, shape)):
                yield f"model.layers.{LAYER}.mlp.experts.{e}.{proj}_proj.weight", m

    path = Path(tempfile.mkdtemp(prefix="umaq_cases_")) / "cases.uqmoepk"
    write_expert_pack(path, stream(), model_id="allenai/OLMoE-1B-7B-0125", model_revision="0" * 40,
                      model_manifest_sha256="0" * 64)
    ref_op.register_moe_forward()
    reader = ExpertPackReader(path)
    handle = ref_op.register_expert_pack(reader)
    run = lambda x, i, w: torch.ops.uma_qmoe.moe_forward(x, i, w, LAYER, handle, False)

    v_x1 = torch.linspace(-0.5, 0.5, 2048, dtype=torch.float32).reshape(1, 2048).to(torch.bfloat16)
    v_idx = torch.arange(8, dtype=torch.int64).reshape(1, 8)
    v_w = torch.full((1, 8), 0.125, dtype=torch.bfloat16)
    v_x32 = torch.linspace(-0.5, 0.5, 32 * 2048, dtype=torch.float32).reshape(32, 2048).to(torch.bfloat16)
    p_x = syn.activations(SEED + 21, p_idx.shape[0])
    d_x = syn.activations(SEED + 22, 1)
    out = {
        "seed": SEED, "layer": LAYER, "hit": np.asarray(hit, np.int64),
        "val_x1_bits": bits(v_x1), "val_idx": v_idx.numpy(), "val_w_bits": bits(v_w),
        "val_y1_bits": bits(run(v_x1, v_idx, v_w)),
        "val_x32_bits": bits(v_x32), "val_y32_bits": bits(run(v_x32, v_idx.repeat(32, 1), v_w.repeat(32, 1))),
        "trace_prefill_idx": p_idx.numpy(), "trace_prefill_w": p_w.numpy(), "trace_prefill_x_bits": bits(p_x),
        "trace_prefill_y_bits": bits(run(p_x, p_idx, p_w)),
        "trace_decode_idx": d_idx.numpy(), "trace_decode_w": d_w.numpy(), "trace_decode_x_bits": bits(d_x),
        "trace_decode_y_bits": bits(run(d_x, d_idx, d_w)),
        "trace_id": trace["trace_id"], "meta": str({"torch": torch.__version__, "numpy": np.__version__}),
    }
    np.savez_compressed(HERE / "reference_cases.npz", **out)
    ref_op.unregister_expert_pack(handle)
    reader.close()
    counts = np.bincount(p_idx.reshape(-1).numpy(), minlength=64)
    print("written", HERE / "reference_cases.npz", "prefill experts hit:", int((counts > 0).sum()), "max", int(counts.max()))


if __name__ == "__main__":
    main()
