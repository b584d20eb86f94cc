"""Benchmark of the routed-expert MoE path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Workload ("step"): one pass of 8192 BF16 N(0,1) tokens through an OLMoE-shaped stack of 16 MoE
layers (hidden 2048, 64 experts, top-8 renormalised, intermediate 1024, W4A16 group-128): per layer
the fused router, the expert-parallel dispatch (N > 1), the grouped-GEMM pipeline and the ordered
combine; the output of a layer, renormalised to unit RMS, is the input of the next.  Weights are
seeded synthetic (no checkpoint); the 3.4 GB of packed weights exceed L2, so every step streams them
from HBM.  With N ranks the experts and the tokens are split N ways (strong scaling); from 4 ranks on a rank's
tokens run as two independent micro-batches on streams of their own (UMAQ_EP_PARTS), one's experts under the
other's exchange.

One JSON line on rank 0.  `value` = tokens/s with inputs resident on the device; `e2e` = the same
through torch.ops.uma_qmoe.moe_forward with every step's activations coming from pinned host memory
and every step's result read back into pinned host memory (the copies ride on a copy stream under the
next step's compute, as in a serving loop); `roofline` / `roofline_down` = the two grouped GEMMs alone
(tensor-bound), `decode` / `decode_qwen` = the batch-1 decode kernels rotating over the layers, replayed
from a CUDA graph (HBM-bound); `cpu_baseline` = the reference's own CPU correctness path (the package
installed under oracle/_ref by oracle/make_ref.py; the port in oracle/ only if that is absent, `kind`
says which) timed on one full-size call of layer 0 on this host.
`--impl reference` times that CPU path as the measured arm.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SEED = 20260917
TOKENS, LAYERS = 8192, 16
DECODE_BYTES = 8 * 3_342_336 + 8_192          # selected experts' codes + scales, x in, y out
QWEN_DECODE_BYTES = 4 * 8_921_088 + 69_206_016 + 4_096 + 8_192     # 4 Q8 experts, the BF16 shared expert + gate, x, y
METRIC, UNIT = "prefill_tokens_per_s", "tokens/s"

# One ncu capture per kernel (dram__bytes_read.sum, dram__bytes_write.sum per launch).  The decode pair was captured
# on the benchmark's own layer; the grouped GEMMs on 2048 tokens of it (a full-size capture would hold more than a
# gigabyte through ~40 replay passes), so their traffic is scaled to the benchmark's token count below.
CAPTURES = {
    "decode_pair": {"read": 17.89e6 + 9.00e6, "write": 0.0},
    # gate/up GEMM fetching its activation rows by index: the read is the layer's gate/up codes and scales (142.6 MB, a
    # few per cent of them L2 hits) plus the 2048 activation rows (8.4 MB); the write is the intermediate
    "gemm_gate_up": {"tokens": 2048, "read": 139.4e6, "write": 19.2e6},
    # down GEMM: weights 71.3 MB + the intermediate rows it reads; the write is the weighted per-route output
    "gemm_down": {"tokens": 2048, "read": 98.4e6, "write": 31.8e6, "weights": 64 * (2048 * 512 + 2048 * 8 * 4)},
}


def gemm_traffic(name: str, tokens: int) -> int:
    """DRAM bytes of one grouped-GEMM launch on `tokens` tokens, from the capture of that kernel: the weights of all
    64 experts are read once whatever the token count; what is written grows with the routes; the gate/up GEMM reads
    each further token's activation row once (4 KiB), the down GEMM its intermediate rows in proportion to the routes."""
    c = CAPTURES[name]
    grow = tokens / c["tokens"]
    if name == "gemm_gate_up":
        return int(c["read"] + (tokens - c["tokens"]) * 2048 * 2 + c["write"] * grow)
    return int(c["weights"] + (c["read"] - c["weights"]) * grow + c["write"] * grow)


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *_):
        if self.proc:
            self.proc.terminate()

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def graphed(fn):
    """Capture `fn` (kernel launches on the current stream only) in a CUDA graph and return a replay
    callable: removes the Python / launch-call overhead from microsecond-scale kernels."""
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return graph.replay


def timed(fn, steps: int, warmup: int, world: int) -> float:
    """Milliseconds per step: CUDA events around `steps` calls, max over ranks."""
    for _ in range(warmup):
        fn()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(stop) / steps], device="cuda")
    if world > 1:
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    return float(ms.item())


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own correctness path (oracle/_ref), else this repository's port of it
# ---------------------------------------------------------------------------------------------

def _layer0_inputs(tokens: int):
    from oracle import moe_oracle as orc
    from uma_qmoe_b200 import synthetic as syn
    shape = syn.OLMOE
    x = syn.activations(SEED, TOKENS)[:tokens].contiguous()
    wr = syn.router_weight(SEED, 0, shape, skew=1.0)
    return orc, syn, shape, x, wr


def reference_layer_call(tokens: int):
    """-> (callable running layer 0 on `tokens` tokens once, kind, cleanup).  kind "reference": the
    UMA-QMoE package installed under oracle/_ref (oracle/make_ref.py) runs its own
    torch.ops.uma_qmoe.moe_forward(..., performance_mode=False) on an ExpertPack its own writer made
    (all 64 experts of layer 0, packed Q4 group-128).  kind "port": oracle/moe_oracle.py."""
    import tempfile
    orc, syn, shape, x, wr = _layer0_inputs(tokens)
    ref_dir = ROOT / "oracle" / "_ref"
    if (ref_dir / "uma_qmoe" / "custom_op.py").exists():
        try:
            sys.path.insert(0, str(ref_dir))
            from uma_qmoe import custom_op as ref_op
            from uma_qmoe.expert_pack import ExpertPackReader, write_expert_pack

            def stream():
                for e in range(shape.experts):
                    for proj, m in zip(("gate", "up", "down"), syn.expert_weights(SEED, 0, e, shape)):
                        yield f"model.layers.0.mlp.experts.{e}.{proj}_proj.weight", m
            tmp = Path(tempfile.mkdtemp(prefix="umaq_ref_"))
            path = tmp / "layer0.uqmoepk"
            write_expert_pack(path, stream(), model_id="allenai/OLMoE-1B-7B-0125", model_revision="0" * 40,
                              model_manifest_sha256="0" * 64)
            ref_op.register_moe_forward()
            reader = ExpertPackReader(path)
            handle = ref_op.register_expert_pack(reader)

            def call():
                # the Hugging Face router's arithmetic (BF16 logits, float32 softmax, top-k, renormalise), then the op
                logits = torch.nn.functional.linear(x, wr)
                probs = torch.softmax(logits, dim=-1, dtype=torch.float)
                w, idx = torch.topk(probs, shape.top_k, dim=-1)
                w = w / w.sum(dim=-1, keepdim=True)
                return torch.ops.uma_qmoe.moe_forward(x, idx, w, 0, handle, False)

            def cleanup():
                ref_op.unregister_expert_pack(handle)
                reader.close()
                path.unlink(missing_ok=True)
            return call, "reference", cleanup
        except Exception as exc:                     # say why the port is used instead
            print(f"bench: oracle/_ref unusable ({type(exc).__name__}: {exc}); timing the port", file=sys.stderr)
    cache: dict[int, tuple] = {}

    def experts(e: int):
        if e not in cache:
            cache[e] = tuple(orc.encode_matrix(m, "q4_group128") for m in syn.expert_weights(SEED, 0, e, shape))
        return cache[e]
    for e in range(shape.experts):
        experts(e)                                  # packing is offline work, not part of the timed call

    def call():
        _pp, ww, ii = orc.router_topk(x, wr, shape.top_k, True)
        return orc.moe_forward(x, ii, ww, experts, num_experts=64, top_k=8, qwen=False)
    return call, "port", lambda: None


def run_cpu(tokens: int, steps: int, warmup: int, budget_s: float) -> dict:
    """Times layer 0 of the stack on `tokens` tokens (one call = the router and the CPU correctness path over
    every hit expert), at most `steps` times and for at most `budget_s` seconds; the step time is that x 16
    layers (the layers are alike; stated as an extrapolation over layers only)."""
    call, kind, cleanup = reference_layer_call(tokens)
    try:
        for _ in range(warmup):
            call()
        times = []
        t_begin = time.perf_counter()
        while len(times) < steps and (not times or time.perf_counter() - t_begin + times[-1] < budget_s):
            t0 = time.perf_counter()
            call()
            times.append(time.perf_counter() - t0)
    finally:
        cleanup()
    per_layer = statistics.median(times)
    return {"value": tokens / (per_layer * LAYERS), "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
            "seconds_per_layer_call": per_layer, "calls_timed": len(times), "sample_tokens": tokens,
            "sample": f"layer 0 of {LAYERS} on {'all ' if tokens == TOKENS else 'the first '}{tokens} of the {TOKENS} tokens "
                      f"(router + CPU correctness path over all 64 experts), {len(times)} call(s) timed, "
                      f"step time = median x {LAYERS} layers (extrapolated over layers only)"}


def cpu_baseline_subprocess() -> dict:
    """One full-size layer-0 call of the CPU arm in a process of its own: the reference package defines the same
    torch.library namespace as the product package, so the two cannot register their operators in one process."""
    cmd = [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0", "--cpu-budget", "60"]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE")}
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        for text in reversed(proc.stdout.strip().splitlines()):
            if text.startswith("{"):
                return json.loads(text)["cpu_baseline"]
        return {"value": None, "unit": UNIT, "error": (proc.stderr or "no output")[-300:]}
    except Exception as exc:
        return {"value": None, "unit": UNIT, "error": f"{type(exc).__name__}: {exc}"[:300]}


def reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    res = run_cpu(args.cpu_tokens, args.steps, min(args.warmup, 1), budget_s=args.cpu_budget)
    line = {"impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": res["calls_timed"], "warmup": min(args.warmup, 1),
            "ms_per_step": res["seconds_per_layer_call"] * 1e3 * LAYERS * (TOKENS / res["sample_tokens"]),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_block(1), "cpu_baseline": res,
            "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def config_block(world: int) -> dict:
    return {"workload": "OLMoE-shaped MoE stack, 16 layers x 8192 tokens, hidden 2048, 64 experts top-8 renormalised, "
                        "intermediate 1024, W4A16 group-128 (expert-parallel prefill)",
            "tokens": TOKENS, "layers": LAYERS, "parallelism": f"ep{world}",
            "l2": "inputs larger than L2 (3.4 GB of packed weights per step)"}


# ---------------------------------------------------------------------------------------------
# native arm
# ---------------------------------------------------------------------------------------------

def native_arm(args) -> None:
    from uma_qmoe_b200 import custom_op, native_backend, ops, synthetic as syn
    from uma_qmoe_b200.stack import MoEStack, rms_renorm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    shape = syn.OLMOE
    mine = range(rank, shape.experts, world)      # interleaved expert placement (ExpertParallelMoE's default)
    backend = native_backend.install_mixed_target_backend()
    # with several ranks the experts of every layer are relabelled so that the interleaved placement is balanced
    stack = MoEStack.build(shape, "q4_group128", LAYERS, SEED, dev, renormalize=True, skew=1.0, experts=mine,
                           balance_ranks=world if os.environ.get("UMAQ_EP_BALANCE", "1") == "1" else 0)
    share = TOKENS // world
    x_host = syn.activations(SEED, TOKENS)[rank * share:(rank + 1) * share].contiguous().pin_memory()
    x_dev = x_host.to(dev)
    out_host = torch.empty_like(x_host).pin_memory()
    launches = 0

    if world == 1:
        class _Stub:
            mapping_count = 1
        handle = custom_op.register_expert_pack(_Stub())
        for l, layer in enumerate(stack.layers):
            backend.preload_layer(handle, l, dev, layer)

        def run_stack(x):
            for l in range(LAYERS):
                w, idx = stack.route(l, x)
                x = rms_renorm(torch.ops.uma_qmoe.moe_forward(x, idx, w, l, handle, True))
            return x
        launches_per_step = LAYERS * 7          # router, sort (2 kernels), gather, 2 grouped GEMMs, combine
    else:
        from uma_qmoe_b200.ep import CudaKernels, ExpertParallelMoE, PeerExchange
        dist = torch.distributed
        # The rank's tokens go through the stack as `parts` independent micro-batches, each on a stream of its own with
        # its own exchange buffer and workspaces: while one part's experts hold the tensor cores, the other part's
        # router, push, barriers and combines (NVLink- and latency-bound) run beside them.  Tokens never interact, so
        # the parts only meet again in the result.
        # Measured (ms per step, 1 | 2 parts): 2 GPUs 8.39 | 8.82 (the halved GEMMs lose more than the overlap wins),
        # 4 GPUs 5.90 | 5.77, 8 GPUs 4.46 | 4.25.
        parts = max(1, int(os.environ.get("UMAQ_EP_PARTS", "2" if world >= 4 else "1")))
        if share % parts:
            parts = 1
        piece = share // parts
        eps_of = [[ExpertParallelMoE(CudaKernels(layer, shape.top_k), shape.experts, shape.top_k) for layer in stack.layers]
                  for _ in range(parts)]
        eps = eps_of[0]
        # Exchange over peer memory (this library's own push / combine kernels on buffers every rank has mapped) when
        # all ranks can map them; otherwise the collective-library exchange (all-gather + all-to-all).
        exs, why = None, ""
        if os.environ.get("UMAQ_EP_EXCHANGE", "peer") == "peer":
            try:
                exs = [PeerExchange(piece, shape.hidden, shape.top_k, rank, world, dev) for _ in range(parts)]
            except Exception as exc:
                why = f"{type(exc).__name__}: {exc}"[:160]
        ok = torch.tensor([1 if exs is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if not int(ok.item()):
            exs, parts, piece = None, 1, share             # the collectives of two parts would have to be ordered
        ex = exs[0] if exs is not None else None
        exchange_name = ("peer memory: rows pushed to the ranks that own one of the token's experts, partial sums written "
                         "into the owner's buffer by the combine kernel, flag barriers (no collective on the data path)"
                         + (f"; {parts} micro-batches of {piece} tokens per rank on streams of their own" if parts > 1 else "")
                         if exs is not None else "all_gather rows + all_to_all partial sums (NCCL)" + (f"; peer mapping failed: {why}" if why else ""))
        dist.barrier()
        side = [torch.cuda.Stream() for _ in range(parts - 1)]

        def part_layer(h, l, x, w, idx):
            return eps_of[h][l].forward_peer(exs[h], x, idx, w) if exs is not None else eps_of[h][l].forward_gather(x, idx, w)

        def on_parts(x, stages, stage):
            """rows = stage(h, i, rows) for i < stages on every part h of x, part h on its own stream; the host issues
            stage i of every part before stage i + 1 of any, so that no part's launches queue up behind another's.
            The results are joined on the current stream."""
            if parts == 1:
                for i in range(stages):
                    x = stage(0, i, x)
                return x
            main = torch.cuda.current_stream()
            streams = [main] + side
            fork = torch.cuda.Event()
            fork.record(main)
            out = torch.empty_like(x)
            rows = [x[h * piece:(h + 1) * piece] for h in range(parts)]
            for s in side:
                s.wait_event(fork)
                x.record_stream(s)
                out.record_stream(s)
            for i in range(stages):
                for h in range(parts):
                    with torch.cuda.stream(streams[h]):
                        rows[h] = stage(h, i, rows[h])
            for h in range(parts):
                with torch.cuda.stream(streams[h]):
                    out[h * piece:(h + 1) * piece].copy_(rows[h])
                    if h:
                        done = torch.cuda.Event()
                        done.record(streams[h])
                        main.wait_event(done)
            return out

        def layer_forward(l, x, w, idx):
            """One layer over all of this rank's tokens through the measured exchange (the parts side by side)."""
            return on_parts(x, 1, lambda h, i, rows: part_layer(h, l, rows, w[h * piece:(h + 1) * piece],
                                                                idx[h * piece:(h + 1) * piece]))

        def run_stack(x):
            def stage(h, l, rows):
                w, idx = stack.route(l, rows)
                return rms_renorm(part_layer(h, l, rows, w, idx))
            return on_parts(x, LAYERS, stage)
        # router; push, barrier, sort (2), 2 GEMMs, combine to peers, barrier, final combine; per part
        launches_per_step = LAYERS * parts * (10 if exs is not None else 8)

    def step_resident():
        run_stack(x_dev)

    def step_in_line():
        """One step with its copies in line: input copy, compute, result copy, host waits."""
        y = run_stack(x_host.to(dev, non_blocking=True))
        out_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed_e2e(steps: int, warmup: int) -> float:
        """Milliseconds per step with every step's input coming from pinned host memory and every step's result
        read back into pinned host memory, as a serving loop runs it: the copies of step i + 1 (in) and of step i
        (out) travel on a copy stream while step i + 1 computes, two device buffers in turn; the host looks at a
        step's result one step later.  Device-timed: from before the first input copy to after the last result copy."""
        main = torch.cuda.current_stream()
        copy = torch.cuda.Stream()
        inputs = [torch.empty_like(x_dev) for _ in range(2)]
        results = [out_host, torch.empty_like(out_host).pin_memory()]
        new_event = lambda: [torch.cuda.Event() for _ in range(2)]
        loaded, computed, stored = new_event(), new_event(), new_event()

        def load(i):                                   # on the copy stream, once step i - 2 no longer reads the buffer
            with torch.cuda.stream(copy):
                if i >= 2:
                    copy.wait_event(computed[i % 2])
                inputs[i % 2].copy_(x_host, non_blocking=True)
                loaded[i % 2].record(copy)

        def loop(n, first=None, last=None):
            if first is not None:
                first.record(copy)
            load(0)
            for i in range(n):
                main.wait_event(loaded[i % 2])
                y = run_stack(inputs[i % 2])
                computed[i % 2].record(main)
                if i + 1 < n:
                    load(i + 1)
                with torch.cuda.stream(copy):
                    copy.wait_event(computed[i % 2])
                    results[i % 2].copy_(y, non_blocking=True)
                    stored[i % 2].record(copy)
                y.record_stream(copy)
                if i >= 1:
                    stored[(i - 1) % 2].synchronize()  # the host has the previous step's result
            if last is not None:
                last.record(copy)
            stored[(n - 1) % 2].synchronize()
        loop(max(1, warmup))
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        loop(steps, start, stop)
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([start.elapsed_time(stop) / steps], device=dev)
        if world > 1:
            torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
        return float(ms.item())

    # The batch-1 decode legs come first: a call is a few microseconds, and right after the long tensor-bound legs
    # the same kernels measured 10 % slower.
    decode_objects, decode_launches, kernel_objects = {}, 0, {}
    if rank == 0 and world == 1 and args.legs == "all":
        decode_objects, decode_launches = decode_legs(stack, x_dev, shape, dev)
        kernel_objects = kernel_legs(stack, x_dev, shape, dev)

    with ClockSampler(local) as clocks:
        ms = timed(step_resident, args.steps, args.warmup, world)
        ms_e2e = timed_e2e(args.steps, max(1, args.warmup // 2))
        ms_in_line = timed(step_in_line, max(2, args.steps // 2), 1, world)

    launches = launches_per_step * args.steps
    pk, pk_kind = peaks()

    line = {"metric": METRIC, "value": TOKENS / (ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_block(world),
            "e2e": {"value": TOKENS / (ms_e2e / 1e3), "unit": UNIT, "ms_per_step": ms_e2e,
                    "ms_per_step_with_copies_in_line": ms_in_line,
                    "copies": "input from and result to pinned host memory every step, on a copy stream under the next step's compute",
                    "h2d_bytes_per_step": x_host.numel() * 2 * world, "d2h_bytes_per_step": x_host.numel() * 2 * world},
            "gpu_launches": launches, "clocks": clocks.summary(),
            **({"exchange": exchange_name} if world > 1 else {}),
            "tflops_step": 65536 * 12_582_912 * LAYERS / (ms / 1e3) / 1e12 / world}

    if rank == 0 and world == 1 and args.legs == "all":
        line.update(kernel_objects)
        line.update(decode_objects)
        # the single-kernel legs (3 x 13 cold launches, ten kernels x 7 graph passes x 8 launches, the 512-token leg:
        # 10 passes x 8 calls x 7 kernels) and the decode legs
        line["gpu_launches"] += 39 + 10 * 7 * 8 + 10 * 8 * 7 + decode_launches
        line["cpu_baseline"] = cpu_baseline_subprocess()
    if world > 1:
        line["ep_check"] = ep_check(stack, eps, ex, layer_forward, x_dev, shape, dev, world)
        line["phases_us"] = ep_phases(stack, eps, ex, x_dev[:piece].contiguous(), shape, dev, world)
        line["phases_us"]["tokens_per_rank_and_micro_batch"] = piece
        if exs is not None:
            line["ep_check"]["barrier_timed_out"] = any(e.timed_out() for e in exs)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


def kernel_legs(stack, x_dev, shape, dev) -> dict:
    """The two grouped GEMMs of layer 0 timed alone (CUDA events around single launches, a 256 MB write between them so
    that the weights come from HBM) against the burst tensor peak, and every kernel of a layer in graphs of eight
    launches.  Run before the long timed region: the peak they are compared with is a burst figure, and after seconds
    at the power cap the same launches take 8 % longer."""
    from uma_qmoe_b200 import ops
    pk, pk_kind = peaks()
    out = {}
    # ---- roofline of the dominant kernel (the gate/up grouped GEMM of layer 0) and of the down GEMM ----
    w, idx = stack.route(0, x_dev)
    routes = ops.route_sort(idx, w, shape.experts)
    xs = ops.gather_rows(x_dev, routes.sorted_route, shape.top_k, permute=True)
    inter = torch.empty((xs.shape[0], shape.intermediate), dtype=torch.bfloat16, device=dev)
    yw = torch.empty((xs.shape[0], shape.hidden), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def cold(fn):
        times = []
        for i in range(3 + 10):
            flush.zero_()                                        # weights leave L2 between launches
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            if i >= 3:
                times.append(a.elapsed_time(b))
        return statistics.mean(times)
    x_perm = ops.gather_rows(x_dev, None, 1, permute=True)        # k order of the quantised kernels, [tokens, H]
    # the gate/up GEMM as the step runs it: activation rows fetched by index, no gathered copy
    gemm_ms = cold(lambda: ops.grouped_gemm_by_index(stack.layers[0], x_perm, routes, shape.top_k, permute_out=True, out=inter))
    gathered_ms = cold(lambda: ops.grouped_gemm(stack.layers[0], 0, xs, routes, permute_out=True, out=inter))
    down_ms = cold(lambda: ops.grouped_gemm(stack.layers[0], 1, inter, routes, route_weight=routes.sorted_weight, out=yw))
    flops = 2.0 * xs.shape[0] * shape.hidden * 2 * shape.intermediate

    def tensor_roofline(kernel, fl, ms_, capture):
        return {"bound": "tensor", "kernel": kernel, "achieved": fl / (ms_ / 1e3) / 1e12, "peak": pk["bf16_tflops"],
                "unit": "TFLOP/s", "frac": fl / (ms_ / 1e3) / 1e12 / pk["bf16_tflops"],
                "traffic": gemm_traffic(capture, TOKENS),
                "traffic_source": f"ncu capture at {CAPTURES[capture]['tokens']} tokens, scaled to {TOKENS} (weights fixed)", "peak_source": f"{pk_kind} (burst)", "ms_per_launch": ms_,
                "flops_per_launch": fl}
    out["roofline"] = tensor_roofline("grouped_gemm_kernel<Q4, gate/up+SwiGLU>, rows fetched by index", flops, gemm_ms, "gemm_gate_up")
    out["roofline"]["ms_per_launch_on_gathered_rows"] = gathered_ms
    out["roofline_down"] = tensor_roofline("grouped_gemm_kernel<Q4, down x route weight>", flops / 2, down_ms, "gemm_down")
    out["kernels_us"] = prefill_kernel_times(stack, x_dev, shape, dev)
    del xs, inter, yw, flush, x_perm
    out["prefill_512_tokens"] = small_prefill_leg(stack, shape, dev)
    return out


def small_prefill_leg(stack, shape, dev) -> dict:
    """One layer on 512 tokens with the skewed router (expert loads vary, some experts get no token): router + the
    whole operator, replayed from a CUDA graph of eight calls."""
    from uma_qmoe_b200 import ops, synthetic as syn
    tokens = 512
    x = syn.activations(SEED + 1, tokens).to(dev)
    wr = syn.router_weight(SEED, 0, shape, skew=1.5).to(dev)
    w, idx = ops.route_topk(x, wr, shape.top_k, True)
    counts = torch.bincount(idx.flatten(), minlength=shape.experts)
    ws = ops.prefill_workspace(stack.layers[0], tokens, shape.top_k, None, dev)

    def eight():
        for _ in range(8):
            ww, ii = ops.route_topk(x, wr, shape.top_k, True)
            ops.moe_prefill(stack.layers[0], x, ii, ww, ws)
    ms = timed(graphed(eight), 5, 2, 1) / 8
    flops = 2.0 * tokens * shape.top_k * 3 * shape.hidden * shape.intermediate
    return {"workload": "one OLMoE layer, 512 tokens, router skew 1.5", "us_per_call": round(ms * 1e3, 2),
            "tokens_per_s": round(tokens / (ms / 1e3)), "tflops": round(flops / (ms / 1e3) / 1e12, 1),
            "experts_without_tokens": int((counts == 0).sum()), "largest_expert_load": int(counts.max())}


def decode_legs(stack, x_dev, shape, dev) -> tuple[dict, int]:
    """The batch-1 decode kernels on the stack's own layers (OLMoE Q4, 16 layers in rotation = 428 MB > L2) and on a
    Qwen1.5-MoE-shaped layer, each replayed from a CUDA graph; beside each the time of a launch that only reads the
    same number of bytes (16-byte loads from many CTAs), i.e. what the part does for a call of that size."""
    from uma_qmoe_b200 import ops
    pk, pk_kind = peaks()

    def hbm_roofline(nbytes, ms_, traffic):
        return {"bound": "hbm", "kernel": "decode_gateup_kernel + decode_down_kernel",
                "achieved": nbytes / (ms_ / 1e3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": nbytes / (ms_ / 1e3) / 1e9 / pk["hbm_gbs"], "traffic": traffic, "peak_source": pk_kind,
                "bytes_per_launch": nbytes}
    steps, warmup = 40, 10
    xd = x_dev[:1].contiguous()
    routes1 = [stack.route(l, xd) for l in range(LAYERS)]
    wsd = ops.decode_workspace(stack.layers[0], shape.top_k, None, dev)
    outd = torch.empty_like(xd)

    def decode_pass():
        for l in range(LAYERS):
            ops.moe_decode(stack.layers[l], xd, routes1[l][1], routes1[l][0], wsd, out=outd)
    dms = timed(graphed(decode_pass), steps, warmup, 1) / LAYERS
    cap = CAPTURES["decode_pair"]
    out = {"decode": {"metric": "decode_hbm_gbs", "workload": "one OLMoE layer call at batch 1: 8 of 64 experts, packed Q4 group-128",
                      "us_per_layer": dms * 1e3, "roofline": hbm_roofline(DECODE_BYTES, dms, int(cap["read"] + cap["write"])),
                      "stream_only_us": stream_floor_us(DECODE_BYTES, LAYERS, dev, steps, warmup),
                      "status": ops.workspace_status(wsd)}}
    out["decode_qwen"] = qwen_decode_leg(dev, hbm_roofline, steps, warmup)
    launches = (2 + 1) * (steps + warmup + 2) * LAYERS + out["decode_qwen"].pop("launches")
    return out, launches


def stream_floor_us(nbytes: int, buffers: int, dev, steps: int, warmup: int) -> float:
    from uma_qmoe_b200 import ops
    nbytes = nbytes // 16 * 16
    bufs = [torch.empty(nbytes, dtype=torch.uint8, device=dev).random_(0, 255) for _ in range(buffers)]

    def run():
        for b in bufs:
            ops.probe_stream(b, 0)
    return timed(graphed(run), steps, warmup, 1) / buffers * 1e3


def qwen_decode_leg(dev, hbm_roofline, steps: int = 20, warmup: int = 3) -> dict:
    """Batch-1 decode of a Qwen1.5-MoE-shaped layer: 4 of 60 Q8 group-128 experts (intermediate 1408), the BF16 shared
    expert (intermediate 5632) and its sigmoid gate; 8 layers in rotation (840 MB > L2), replayed from a CUDA graph."""
    from uma_qmoe_b200 import ops, synthetic as syn
    from uma_qmoe_b200.stack import MoEStack, random_shared_expert
    layers, shape = 8, syn.QWEN
    stack = MoEStack.build(shape, "q8_group128", layers, SEED, dev, renormalize=False, skew=1.0)
    shared = [random_shared_expert(shape, SEED + l, dev) for l in range(layers)]
    x = syn.activations(SEED, 1).to(dev)
    routes = [stack.route(l, x) for l in range(layers)]
    ws = ops.decode_workspace(stack.layers[0], shape.top_k, shared[0], dev)
    out = torch.empty_like(x)

    def run():
        for l in range(layers):
            ops.moe_decode(stack.layers[l], x, routes[l][1], routes[l][0], ws, shared[l], out=out)
    ms = timed(graphed(run), steps, warmup, 1) / layers
    return {"metric": "decode_hbm_gbs", "workload": "one Qwen1.5-MoE layer call at batch 1: 4 of 60 experts Q8 group-128, "
            "BF16 shared expert + gate", "us_per_layer": ms * 1e3, "roofline": hbm_roofline(QWEN_DECODE_BYTES, ms, None),
            "stream_only_us": stream_floor_us(QWEN_DECODE_BYTES, layers, dev, steps, warmup),
            "status": ops.workspace_status(ws), "launches": (2 + 1) * (steps + warmup + 2) * layers}


def prefill_kernel_times(stack, x, shape, dev) -> dict:
    """Device time (microseconds) of every kernel of one prefill layer on the tokens of `x` (layer 0), each replayed
    from a CUDA graph of 8 back-to-back launches so that no launch gap is inside the figure."""
    from uma_qmoe_b200 import ops
    from uma_qmoe_b200.stack import rms_renorm
    layer = stack.layers[0]
    w, idx = stack.route(0, x)
    routes = ops.route_sort(idx, w, shape.experts)
    xs = ops.gather_rows(x, routes.sorted_route, shape.top_k, permute=True)
    x_perm = ops.gather_rows(x, None, 1, permute=True)
    inter = torch.empty((xs.shape[0], shape.intermediate), dtype=torch.bfloat16, device=dev)
    yw = torch.empty((xs.shape[0], shape.hidden), dtype=torch.bfloat16, device=dev)
    ws = ops.prefill_workspace(layer, x.shape[0], shape.top_k, None, dev)
    phases = [("router", lambda: stack.route(0, x)),
              ("route_sort", lambda: ops.route_sort(idx, w, shape.experts)),
              ("permute_k", lambda: ops.gather_rows(x, None, 1, permute=True)),
              ("gemm_gate_up", lambda: ops.grouped_gemm_by_index(layer, x_perm, routes, shape.top_k, permute_out=True, out=inter)),
              ("gather_rows_not_on_the_path", lambda: ops.gather_rows(x, routes.sorted_route, shape.top_k, permute=True)),
              ("gemm_gate_up_on_gathered_rows", lambda: ops.grouped_gemm(layer, 0, xs, routes, permute_out=True, out=inter)),
              ("gemm_down", lambda: ops.grouped_gemm(layer, 1, inter, routes, route_weight=routes.sorted_weight, out=yw)),
              ("combine", lambda: ops.combine_routes(yw, idx, routes.route_pos)),
              ("rms_norm", lambda: rms_renorm(x)),
              ("whole_operator", lambda: ops.moe_prefill(layer, x, idx, w, ws))]
    out = {}
    for name, fn in phases:
        def eight(fn=fn):
            for _ in range(8):
                fn()
        out[name] = round(timed(graphed(eight), 3, 1, 1) / 8 * 1e3, 2)
    return out


def compare(got: torch.Tensor, want: torch.Tensor) -> dict:
    a, b = got.double().flatten(), want.double().flatten()
    return {"max_abs": float((a - b).abs().max()), "cosine": float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-300))}


def ep_check(stack, eps, ex, layer_forward, x_dev, shape, dev, world) -> dict:
    """Outside the timed region: layer 0 over this rank's tokens through the measured exchange and through the
    exact-count exchange, against the one-GPU operator on the same tokens with the full layer 0 (every rank builds
    it from the same seeds).  Worst case over the ranks."""
    from uma_qmoe_b200 import ops
    from uma_qmoe_b200.stack import random_layer
    dist = torch.distributed
    full = random_layer(shape, "q4_group128", SEED, dev, stack.orders[0])      # the whole layer 0, same labels
    w, idx = stack.route(0, x_dev)
    ws = ops.prefill_workspace(full, x_dev.shape[0], shape.top_k, None, dev)
    want = ops.moe_prefill(full, x_dev, idx, w, ws)
    got = layer_forward(0, x_dev, w, idx)
    exact = eps[0].forward(x_dev, idx, w)
    torch.cuda.synchronize()
    m = compare(got, want)
    stats = torch.tensor([m["max_abs"], -m["cosine"], 0.0 if torch.equal(exact, want) else 1.0], device=dev, dtype=torch.float64)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    del full, ws
    return {"max_abs": float(stats[0]), "cosine": float(-stats[1]), "bit_equal_exact_path": bool(stats[2] == 0),
            "tolerance": "max_abs <= 2e-2, cosine >= 0.9999 against the one-GPU operator", "layer": 0,
            "pass": bool(stats[0] <= 2e-2 and -stats[1] >= 0.9999 and stats[2] == 0)}


def ep_phases(stack, eps, ex, x_dev, shape, dev, world) -> dict:
    """CUDA-event time of every phase of one layer's expert-parallel step (layer 0, median of 5, max over ranks)."""
    from uma_qmoe_b200.stack import rms_renorm
    dist = torch.distributed
    ep = eps[0]
    ops = ep.kernels.ops
    w, idx = stack.route(0, x_dev)
    if ex is not None:
        phases = [("router", lambda: stack.route(0, x_dev)),
                  ("push", lambda: ep.peer_push(ex, x_dev, idx, w)),
                  ("barrier_1", lambda: ops.ep_barrier(ex.peers, ex.off_flags, ex.epoch, ex.status)),
                  ("local_experts_and_combine_to_peers", lambda: ep.peer_compute(ex)),
                  ("barrier_2", lambda: ops.ep_barrier(ex.peers, ex.off_flags, ex.epoch, ex.status)),
                  ("final_combine", lambda: ep.peer_combine(ex)),
                  ("rms_norm", lambda: rms_renorm(x_dev))]
    else:
        phases = [("router", lambda: stack.route(0, x_dev)),
                  ("whole_layer_all_gather_local_experts_all_to_all_combine", lambda: ep.forward_gather(x_dev, idx, w)),
                  ("rms_norm", lambda: rms_renorm(x_dev))]
    times = {name: [] for name, _ in phases}
    for rep in range(6):
        dist.barrier()
        torch.cuda.synchronize()
        for name, fn in phases:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(400_000)          # ~0.2 ms of device idle time, so the host's launch calls are not in the figure
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            if rep:
                times[name].append(a.elapsed_time(b) * 1e3)
    med = torch.tensor([statistics.median(times[name]) for name, _ in phases], device=dev, dtype=torch.float64)
    dist.all_reduce(med, op=dist.ReduceOp.MAX)
    out = {name: round(float(v), 1) for (name, _), v in zip(phases, med)}
    if ex is not None:
        # bytes this rank writes into other ranks' buffers per layer: rows to owners of the token's experts + routes
        sent = int((ex.present >= 0).sum().item()) - int((ex.present[:, ep.rank] >= 0).sum().item())
        out["push_bytes"] = sent * shape.hidden * 2 + (world - 1) * x_dev.shape[0] * shape.top_k * 8
        out["push_gbs"] = round(out["push_bytes"] / (out["push"] * 1e-6) / 1e9, 1) if out["push"] else None
        out["nvlink_peak_gbs_per_direction"] = 900
    return out


def kernel_case(args) -> None:
    """A small case of one kernel, sized for a profiler capture: a few launches, < 1 GB on the device."""
    from uma_qmoe_b200 import ops, synthetic as syn
    from uma_qmoe_b200.stack import MoEStack

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.only == "model":
        return model_case(args, dev)
    if args.only == "phases":
        return prefill_phases_case(args, dev)
    if args.only == "stream":
        return stream_case(args, dev)
    if args.only == "stage":
        return stage_case(args, dev)
    qwen = args.model == "qwen"
    shape = syn.QWEN if qwen else syn.OLMOE
    encoding = args.encoding or ("q8_group128" if qwen else "q4_group128")
    stack = MoEStack.build(shape, encoding, args.layers if args.only == "decode" else 1, SEED, dev,
                           renormalize=not qwen, skew=1.0)
    if args.only == "decode":
        # an OLMoE layer (Q4) or a Qwen1.5-MoE layer (Q8 routed experts, BF16 shared expert + gate)
        from uma_qmoe_b200.stack import random_shared_expert
        shared = [random_shared_expert(shape, SEED + l, dev) for l in range(args.layers)] if qwen else None
        nbytes = QWEN_DECODE_BYTES if qwen else DECODE_BYTES
        x = syn.activations(SEED, 1).to(dev)
        routes = [stack.route(l, x) for l in range(args.layers)]
        ws = ops.decode_workspace(stack.layers[0], shape.top_k, shared[0] if qwen else None, dev)
        out = torch.empty_like(x)

        def run():
            for l in range(args.layers):
                ops.moe_decode(stack.layers[l], x, routes[l][1], routes[l][0], ws, shared[l] if qwen else None, out=out)
        ms = timed(run, args.steps, args.warmup, 1) / args.layers
        msg = timed(graphed(run), args.steps, args.warmup, 1) / args.layers
        print(json.dumps({"case": "decode", "model": args.model, "bytes_per_layer": nbytes,
                          "us_per_layer_eager": ms * 1e3, "us_per_layer": msg * 1e3,
                          "gbs": nbytes / (msg / 1e3) / 1e9, "status": ops.workspace_status(ws)}))
    else:
        x = syn.activations(SEED, args.tokens).to(dev)
        quant = encoding != "bf16_le"               # quantised GEMMs take their activations in the permuted k order
        w, idx = stack.route(0, x)
        routes = ops.route_sort(idx, w, shape.experts)
        xs = ops.gather_rows(x, routes.sorted_route, shape.top_k, permute=quant)
        inter = torch.empty((xs.shape[0], shape.intermediate), dtype=torch.bfloat16, device=dev)
        yw = torch.empty((xs.shape[0], shape.hidden), dtype=torch.bfloat16, device=dev)

        source = ops.gather_rows(x, None, 1, permute=True) if quant else x     # [tokens, H] for the by-index kernel

        def gate_up():
            if args.by_index:
                ops.grouped_gemm_by_index(stack.layers[0], source, routes, shape.top_k, permute_out=quant, out=inter)
            else:
                ops.grouped_gemm(stack.layers[0], 0, xs, routes, permute_out=quant, out=inter, variant=args.variant)

        def run():
            gate_up()
            ops.grouped_gemm(stack.layers[0], 1, inter, routes, route_weight=routes.sorted_weight, out=yw,
                             variant=args.variant)
        ms = timed(run, args.steps, args.warmup, 1)
        ms1 = timed(gate_up, args.steps, args.warmup, 1)
        ms2 = timed(lambda: ops.grouped_gemm(stack.layers[0], 1, inter, routes, route_weight=routes.sorted_weight,
                                             out=yw, variant=args.variant), args.steps, args.warmup, 1)
        flops = 2.0 * xs.shape[0] * 3 * shape.hidden * shape.intermediate
        print(json.dumps({"case": "gemm", "model": args.model, "encoding": encoding, "tokens": args.tokens, "variant": args.variant,
                          "gate_up_rows_by_index": bool(args.by_index), "ms_both_gemms": ms, "ms_gate_up": ms1, "ms_down": ms2,
                          "tflops": flops / (ms / 1e3) / 1e12, "tflops_gate_up": flops * 2 / 3 / (ms1 / 1e3) / 1e12,
                          "tflops_down": flops / 3 / (ms2 / 1e3) / 1e12, "status": int(routes.status.item())}))


def stream_case(args, dev) -> None:
    """Floors for the batch-1 decode call of --model: (a) launches that only read the call's bytes (16-byte loads
    from many CTAs; bulk copies into a shared-memory ring from one CTA per SM), (b) the decode kernels themselves
    with their arithmetic and / or their weight copies switched off.  Same harness as the decode figure: the layers'
    buffers in rotation (more bytes than L2), replayed from a CUDA graph, CUDA events."""
    from uma_qmoe_b200 import ops
    qwen = args.model == "qwen"
    nbytes = (QWEN_DECODE_BYTES if qwen else DECODE_BYTES) // 16 * 16
    layers = 8 if qwen else 16
    pk, pk_kind = peaks()
    bufs = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device=dev) for _ in range(layers)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = {"case": "stream", "model": args.model, "bytes_per_launch": nbytes, "peak_gbs": pk["hbm_gbs"], "peak_source": pk_kind}
    for mode, name in ((0, "loads_16_bytes_many_ctas"), (1, "bulk_copy_ring_one_cta_per_sm")):
        def run(mode=mode):
            for b in bufs:
                ops.probe_stream(b, mode, status)
        ms = timed(graphed(run), args.steps, args.warmup, 1) / layers
        out[name] = {"us_per_launch": round(ms * 1e3, 2), "gbs": round(nbytes / (ms / 1e3) / 1e9, 1),
                     "frac_of_peak": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3)}
    out["probe_status"] = int(status.item())
    # the switch is read once per process, so each setting runs in a process of its own
    for flag, name in ((3, "decode_kernels_without_weight_copies_and_arithmetic"), (1, "decode_kernels_without_arithmetic"),
                       (0, "decode_kernels")):
        cmd = [sys.executable, str(ROOT / "bench.py"), "--only", "decode", "--model", args.model, "--layers", str(layers),
               "--steps", str(args.steps), "--warmup", str(args.warmup)]
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, UMAQ_DECODE_DEBUG=str(flag)))
        lines = [t for t in proc.stdout.splitlines() if t.startswith("{")]
        out[name] = {"us_per_layer": round(json.loads(lines[-1])["us_per_layer"], 2)} if lines else {"error": proc.stderr[-200:]}
    print(json.dumps(out))


def stage_case(args, dev) -> None:
    """Host -> device staging of one OLMoE layer (64 experts, packed Q4: 213.9 MB) from an ExpertPack file: the
    native reader (C++ mapping and checks, worker thread, pinned 32 MiB chunks, one cudaMemcpyAsync per piece) against
    the Python reader's path (pinned tensors filled expert by expert, then copied).  The file is written by this
    package's writer from a layer packed on the device; the staged bytes must equal that layer's."""
    import tempfile
    from uma_qmoe_b200 import custom_op, native_backend, synthetic as syn
    from uma_qmoe_b200.formats import PackedTensor
    from uma_qmoe_b200.pack_files import ExpertPackFile, NativeExpertPackFile
    from uma_qmoe_b200.pack_writer import write_expert_pack
    from uma_qmoe_b200.packs import expert_tensor_name
    from uma_qmoe_b200.stack import random_layer
    shape = syn.OLMOE
    source = random_layer(shape, "q4_group128", SEED, dev)
    host = {p: (getattr(source, p).cpu().numpy().reshape(shape.experts, -1), getattr(source, p + "_scales").cpu().numpy().reshape(shape.experts, -1))
            for p in ("gate", "up", "down")}

    def tensors():
        for e in range(shape.experts):
            for p in ("gate", "up", "down"):
                dims = (shape.hidden, shape.intermediate) if p == "down" else (shape.intermediate, shape.hidden)
                yield expert_tensor_name(0, e, p + "_proj"), PackedTensor("q4_group128", dims, host[p][0][e].tobytes(), host[p][1][e].tobytes())
    tmp = Path(tempfile.mkdtemp(prefix="umaq_stage_"))
    path = tmp / "layer0.uqmoepk"
    identity = dict(model_id="allenai/OLMoE-1B-7B-0125", model_revision="0" * 40, model_manifest_sha256="0" * 64)
    t0 = time.perf_counter()
    info = write_expert_pack(path, tensors(), **identity)
    write_s = time.perf_counter() - t0
    backend = native_backend.install_mixed_target_backend()
    out = {"case": "stage", "layer_bytes": source.device_storage_bytes, "file_bytes": info["file_size"], "write_seconds": round(write_s, 3)}
    for name, cls in (("native_reader", NativeExpertPackFile), ("python_reader", ExpertPackFile)):
        t0 = time.perf_counter()
        reader = cls(path, expected_model_id=identity["model_id"])
        open_s = time.perf_counter() - t0
        times = []
        for rep in range(3):
            handle = custom_op.register_expert_pack(reader)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            with custom_op.acquire_expert_pack(handle) as r:
                layer = backend._device_layer(handle, 0, dev, r, "olmoe")
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
            same = all(torch.equal(a.reshape(-1).view(torch.uint8), b.reshape(-1).view(torch.uint8))
                       for a, b in zip(layer.tensors, source.tensors))
            custom_op.unregister_expert_pack(handle)          # drops the staged copy
        best = min(times)
        out[name] = {"open_and_validate_seconds": round(open_s, 3), "stage_seconds": [round(t, 4) for t in times],
                     "gb_per_s": round(source.device_storage_bytes / best / 1e9, 2), "bytes_equal": bool(same)}
        reader.close()
    path.unlink()
    tmp.rmdir()
    print(json.dumps(out))


def prefill_phases_case(args, dev) -> None:
    """Device time of every kernel of one prefill layer (OLMoE Q4, layer 0, --tokens tokens)."""
    from uma_qmoe_b200 import synthetic as syn
    from uma_qmoe_b200.stack import MoEStack
    shape = syn.OLMOE
    stack = MoEStack.build(shape, "q4_group128", 1, SEED, dev, renormalize=True, skew=1.0)
    x = syn.activations(SEED, args.tokens).to(dev)
    print(json.dumps({"case": "phases", "tokens": args.tokens, "us": prefill_kernel_times(stack, x, shape, dev)}))


def model_case(args, dev) -> None:
    """A Qwen1.5-MoE-A2.7B-shaped model with random weights (24 layers unless --layers says
    otherwise), experts of layers 0-15 BF16 and 16-23 Q8 (`--variant 0`) or all Q4 (`--variant 1`), greedy decode of
    128 prompt tokens + 32 generated at batch 1 through the Hugging Face model with this package's blocks."""
    import transformers
    from uma_qmoe_b200.host import greedy_decode, greedy_decode_graphed, install_quantized_blocks
    layers = args.layers if args.layers != 2 else 24
    cfg = transformers.Qwen2MoeConfig(vocab_size=151936, hidden_size=2048, num_hidden_layers=layers,
                                      num_attention_heads=16, num_key_value_heads=16, max_position_embeddings=8192,
                                      intermediate_size=5632, moe_intermediate_size=1408,
                                      shared_expert_intermediate_size=5632, num_experts=60, num_experts_per_tok=4,
                                      norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[])
    torch.manual_seed(SEED)
    with torch.device(dev):
        model = transformers.Qwen2MoeForCausalLM(cfg).to(torch.bfloat16).eval()
    policy = ("q4_group128" if args.variant == 1 else
              {i: ("bf16_le" if i < layers * 2 // 3 else "q8_group128") for i in range(layers)})
    host = install_quantized_blocks(model, policy)
    prompt = torch.randint(0, cfg.vocab_size, (1, 128), generator=torch.Generator().manual_seed(SEED)).to(dev)
    greedy_decode(model, prompt, 4)                                  # warm-up: workspaces, autotuned attention
    runs = [greedy_decode(model, prompt, 32) for _ in range(3)]
    tpot = sorted(t for r in runs for t in r["tpot_ms"])
    graph_stats = {}
    try:                                            # the same loop with the decode step replayed from a CUDA graph
        first = greedy_decode_graphed(model, prompt, 32)
        more = [greedy_decode_graphed(model, prompt, 32, decoder=first["decoder"]) for _ in range(3)]
        gt = sorted(t for r in more for t in r["tpot_ms"])
        graph_stats = {"graphed_tpot_ms_p50": statistics.median(gt), "graphed_tpot_ms_p95": gt[int(0.95 * (len(gt) - 1))],
                   "graphed_decode_tokens_per_s": 1e3 / statistics.median(gt),
                   "graphed_ttft_ms": statistics.median(r["ttft_ms"] for r in more),
                   "graphed_tokens_equal_eager": more[0]["tokens"] == runs[0]["tokens"]}
    except Exception as exc:
        graph_stats = {"graphed": f"capture failed: {type(exc).__name__}: {exc}"[:300]}
    # the MoE blocks alone (router, routed experts, shared expert and gate of every layer) on one token, replayed from a
    # CUDA graph: their share of the time per generated token
    h = torch.randn(1, 1, cfg.hidden_size, device=dev, dtype=torch.bfloat16)

    @torch.no_grad()
    def blocks_only():
        for layer in model.model.layers:
            layer.mlp(h)
    moe_ms = timed(graphed(blocks_only), 20, 5, 1)
    graph_stats["moe_blocks_ms_per_token"] = moe_ms
    if "graphed_tpot_ms_p50" in graph_stats:
        graph_stats["moe_share_of_graphed_tpot"] = moe_ms / graph_stats["graphed_tpot_ms_p50"]
    print(json.dumps({"case": "model", "layers": layers, "policy": "all q4_group128" if args.variant == 1 else
                      "layers 0-15 bf16_le, 16-23 q8_group128", "prompt_tokens": 128, "new_tokens": 32,
                      "ttft_ms": statistics.median(r["ttft_ms"] for r in runs), "tpot_ms_p50": statistics.median(tpot),
                      "tpot_ms_p95": tpot[int(0.95 * (len(tpot) - 1))], "decode_tokens_per_s": 1e3 / statistics.median(tpot),
                      "expert_storage_bytes": host.evidence["expert_storage_bytes"],
                      "tokens_equal_across_runs": all(r["tokens"] == runs[0]["tokens"] for r in runs), **graph_stats}))
    host.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("native", "reference"), default="native")
    ap.add_argument("--cpu-tokens", type=int, default=TOKENS, help="tokens of the CPU arm's layer-0 call")
    ap.add_argument("--cpu-budget", type=float, default=240.0, help="seconds the CPU arm may spend on timed calls")
    ap.add_argument("--legs", choices=("all", "none"), default="all",
                    help="none: only the timed step (for a profiler's launch list); the line then lacks roofline, decode and cpu_baseline")
    ap.add_argument("--only", choices=("all", "decode", "gemm", "model", "phases", "stream", "stage"), default="all",
                    help="small single-kernel cases for profiler captures (not a bench line)")
    ap.add_argument("--tokens", type=int, default=1024, help="tokens of the --only gemm case")
    ap.add_argument("--layers", type=int, default=2, help="layers of the --only cases")
    ap.add_argument("--model", choices=("olmoe", "qwen"), default="olmoe",
                    help="layer shape of the --only decode case: olmoe = config 0 (Q4), qwen = config 2 (Q8 + shared)")
    ap.add_argument("--encoding", choices=("q4_group128", "q8_group128", "bf16_le"), default=None,
                    help="expert encoding of the --only decode / gemm cases (default: q4 for olmoe, q8 for qwen)")
    ap.add_argument("--by-index", action="store_true",
                    help="--only gemm: the gate/up GEMM fetches its activation rows by index (as the operator runs it)")
    ap.add_argument("--variant", type=int, default=0, choices=(0, 1, 2),
                    help="grouped GEMM kernel of the --only gemm case: 0/1 one CTA per tile (default), 2 CTA pairs")
    args = ap.parse_args()
    if args.only != "all":
        kernel_case(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        native_arm(args)


if __name__ == "__main__":
    main()
