#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second of a Qwen2 1.5B-class model
(random weights, bfloat16) at batch 8 and a 4,096-token context, with prefill, roofline and
batch-1 / batch-64 points on the same JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  Each request holds a 2,048-token prompt and
decodes towards the 4,096-token context; the K timed steps are centred on the middle of that
range (context 3,072), so their cost is the workload's mean.  ``value`` times the device alone
(the captured decode step replayed back to back, greedy choice on the device); ``e2e`` times the
same steps through ``InferenceEngine.step()``, host token lists in, sampled tokens out, with the
step's descriptor copied from pinned memory and the chosen tokens read back every step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_1P5B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 8960, "vocab_size": 151936, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 4096, "torch_dtype": "bfloat16",
}
SEED = 3
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE_SIZE = 16


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    if os.path.isfile(path):
        try:
            with open(path) as f:
                j = json.load(f)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(j.get(k), (int, float)):
                    out[k] = float(j[k])
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,clocks.mem,power.draw")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons, mem, watts = [], 0, set(), [], []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                mhz.append(int(float(s[0])))
                mx = max(mx, int(float(s[1])))
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
            for column, into in ((6, mem), (7, watts)):          # memory clock and power: what the SM clock does not show
                try:
                    into.append(float(s[column]))
                except (ValueError, IndexError):
                    pass
        mhz.sort(), mem.sort(), watts.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz),
                "mem_mhz": int(mem[len(mem) // 2]) if mem else None, "watts": int(watts[len(watts) // 2]) if watts else None}


def weight_bytes_per_step(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (qd + 2 * kd) * h + (qd + 2 * kd) + h * qd + 2 * i * h + h * i + 2 * h
    return 2 * (layers * per_layer + v * h + h)


def kv_bytes_per_token(cfg, layers):
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, n):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kd = cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = layers * ((qd + 2 * kd) * h + h * qd + 3 * i * h)
    attn = layers * 4 * qd * (n * (n + 1) // 2)          # QK^T and PV over the causal half
    return 2 * n * linear + attn + 2 * v * h


def random_prompts(batch, n, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, n), generator=g).tolist()


def measure_prefill(core, cfg, layers, warmup, reps, pk):
    import torch
    from zedinfer_b200.engine.core import StepEntry
    prompts = random_prompts(warmup + reps, PROMPT_LEN, cfg["vocab_size"], SEED + 100)
    times = []
    for i, ids in enumerate(prompts):
        rid = ("prefill", i)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        core.step([StepEntry(rid, ids, [PROMPT_LEN - 1])])
        b.record()
        torch.cuda.synchronize()
        core.end(rid)
        if i >= warmup:
            times.append(a.elapsed_time(b))
    ms = sum(times) / len(times)
    flops = prefill_flops(cfg, layers, PROMPT_LEN)
    return {"value": round(PROMPT_LEN / ms * 1000.0, 1), "tokens": PROMPT_LEN, "ms": round(ms, 3),
            "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}


def prefill_requests(core, prompts, tag):
    """Put the prompts into the cache (one request per step) and return ids, first tokens and request caches."""
    import torch
    from zedinfer_b200 import ops
    from zedinfer_b200.engine.core import StepEntry
    rids, first = [], []
    out = torch.empty(1, dtype=torch.int32, device=core.device)
    for i, ids in enumerate(prompts):
        rid = (tag, i)
        logits = core.step([StepEntry(rid, ids, [len(ids) - 1])])
        ops.argmax(logits, out)
        first.append(int(out.item()))
        rids.append(rid)
    return rids, first


def measure_decode_device(core, cfg, batch, steps, warmup):
    """Device-only decode: the captured step with greedy choice and hand-over, replayed back to back."""
    import torch
    prompts = random_prompts(batch, PROMPT_LEN, cfg["vocab_size"], SEED + batch)
    rids, first = prefill_requests(core, prompts, f"dev{batch}")
    rcs = [core.request(r) for r in rids]
    start = decode_start(steps, warmup)
    total_new = (start - PROMPT_LEN) + warmup + steps
    for rc in rcs:
        core.cache.ensure(rc, rc.length + total_new + 1)
    g = core.decode_graph(batch, greedy=True, longest=max(rc.length for rc in rcs) + total_new + 1)
    g.fill(first, rcs)
    for _ in range(start - PROMPT_LEN):
        g.replay()
    for _ in range(warmup):
        g.replay()
    # exactly `steps` steps between the first and the last event; events in between cut them into a few regions
    # whose rates give the spread (an event costs nothing that a step would notice)
    cuts = region_cuts(steps)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(len(cuts) + 1)]
    torch.cuda.synchronize()
    events[0].record()
    done = 0
    for k, upto in enumerate(cuts):
        for _ in range(upto - done):
            g.replay()
        done = upto
        events[k + 1].record()
    torch.cuda.synchronize()
    ms = events[0].elapsed_time(events[-1]) / steps
    per_region = [events[k].elapsed_time(events[k + 1]) / (cuts[k] - (cuts[k - 1] if k else 0)) for k in range(len(cuts))]
    for rid in rids:
        core.end(rid)
    mean_ctx = start + warmup + steps / 2.0
    return {"tok_s": batch * 1000.0 / ms, "ms": ms, "mean_ctx": mean_ctx, "launches": g.launches * steps,
            "spread": spread(per_region)}


def region_cuts(steps, regions=5):
    """Step counts at which the timed steps are cut into (at most) ``regions`` regions of equal length."""
    regions = max(1, min(regions, steps))
    return [steps * (k + 1) // regions for k in range(regions)]


def spread(per_region_ms):
    v = sorted(per_region_ms)
    return {"regions": len(v), "ms_min": round(v[0], 4), "ms_median": round(v[len(v) // 2], 4), "ms_max": round(v[-1], 4)}


def measure_decode_e2e(core, cfg, batch, steps, warmup, run_ahead=True):
    """The same steps through the public entry point: sampled tokens out every step.  With ``run_ahead`` (the
    engine's default) a decode step takes its input tokens on the device from the step before and the host reads
    each step's tokens while the next one runs; without it the host sends every step's tokens itself."""
    import torch
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine, InferenceRequest, RequestPhase
    sc = SchedulerConfig(max_batch_tokens=4096, max_prefill_tokens=2048, max_batch_requests=max(batch, 1),
                         kv_block_size=PAGE_SIZE, cuda_graphs=True, run_ahead=run_ahead)
    engine = InferenceEngine(core, sc)
    prompts = random_prompts(batch, PROMPT_LEN, cfg["vocab_size"], SEED + batch)
    gen = GenerationConfig(max_new_tokens=CONTEXT - PROMPT_LEN, use_argmax=True, ignore_eos=True)
    reqs = [InferenceRequest(p, gen) for p in prompts]
    for r in reqs:
        engine.submit_async(r)
    while any(r.phase != RequestPhase.DECODE for r in reqs):
        engine.step()
    mid = (PROMPT_LEN + CONTEXT) // 2
    start = max(PROMPT_LEN + 1, min(mid - steps // 2, CONTEXT - steps - warmup - 2))
    while len(reqs[0].output_ids) + PROMPT_LEN < start:
        engine.step()
    for _ in range(warmup):
        engine.step()
    h2d0 = core._ring.bytes_staged
    cuts = region_cuts(steps)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    stamps, done = [t0], 0
    for upto in cuts:                                # the host's clock at a few places on the way: the spread
        for _ in range(upto - done):
            engine.step()
        done = upto
        stamps.append(time.perf_counter())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    per_region = [(stamps[k + 1] - stamps[k]) * 1000.0 / (cuts[k] - (cuts[k - 1] if k else 0)) for k in range(len(cuts))]
    h2d = (core._ring.bytes_staged - h2d0) / steps
    for r in reqs:
        engine.scheduler.cancel(r)
    while engine.has_work():
        engine.step()
    for r in reqs:
        core.end(r.request_id)
    return {"tok_s": batch * steps / dt, "ms": dt * 1000.0 / steps, "h2d": int(h2d), "d2h": 4 * (batch + 1),      # the tokens and the kernels' status word
            "spread": spread(per_region)}


def measure_head(core, cfg, rows, reps=20):
    """Milliseconds of the output head's product alone at `rows` rows (its weight is larger than L2, so every call
    streams it from memory): what the step's time and bytes are reduced by for the figure without the head."""
    import torch
    x = (torch.randn(rows, cfg["hidden_size"], device=core.device) * 0.5).to(torch.bfloat16)
    logits = torch.empty(rows, cfg["vocab_size"], dtype=torch.float32, device=core.device)
    for _ in range(3):
        core.model.head.forward(x, logits)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(reps):
        core.model.head.forward(x, logits)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


REF_BENCH = os.path.join(ROOT, "baseline", "_ref", "ref_bench")


def decode_start(steps, warmup):
    mid = (PROMPT_LEN + CONTEXT) // 2
    return max(PROMPT_LEN, min(mid - steps // 2, CONTEXT - steps - warmup - 1))


def reference_arm(args):
    """The same metric and sizes on tianyuxbear/zedinfer's own NVIDIA path: ``baseline/_ref/ref_bench`` is the
    reference's unmodified transformer_forward, paged context, block pool, CUDA kernels, cuBLASLt product and
    FlashInfer wrappers, compiled by ``baseline/ref_bench/build.py`` and driven as its profiler and serving loop drive
    them (random bfloat16 weights of the same shapes, its own argmax sampler reading every request's token back each
    step).  Nothing of zedinfer_b200 runs in this arm."""
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    if args.gpus != 1:
        return unavailable("the reference runs on one GPU")
    if not (os.path.isfile(REF_BENCH) and os.access(REF_BENCH, os.X_OK)):
        return unavailable("baseline/_ref/ref_bench is not built: tianyuxbear/zedinfer has no Python package to install "
                           "(an xmake C++ project with empty submodules); `python baseline/ref_bench/build.py <checkout>` "
                           "compiles its NVIDIA path with nvcc")
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    cfg = dict(MODEL_1P5B, num_hidden_layers=args.layers)
    pk = peaks()
    start = decode_start(steps, warmup)
    pts = [] if args.no_points else [1, 64]
    jobs = [f"prefill:{PROMPT_LEN}:5:3", f"decode:{args.batch}:{start}:{steps}:{warmup}"]
    jobs += [f"decode:{b}:{decode_start(min(steps, 128), warmup)}:{min(steps, 128)}:{warmup}" for b in pts]
    cmd = [REF_BENCH] + [str(cfg[k]) for k in ("num_hidden_layers", "hidden_size", "intermediate_size", "vocab_size",
                                                "num_attention_heads", "num_key_value_heads", "head_dim", "rope_theta",
                                                "rms_norm_eps")] + [str(PAGE_SIZE)] + jobs
    clocks = ClockSampler()
    clocks.start()
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    except subprocess.TimeoutExpired:
        clocks.stop()
        return unavailable("the reference's run did not end within 25 minutes")
    clocks.stop()
    rows = [ln.split() for ln in proc.stdout.splitlines() if ln.split() and ln.split()[0] in ("prefill", "decode")]
    if proc.returncode != 0 or len(rows) != len(jobs):
        tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or ["no output"]
        return unavailable(f"the reference's own run failed (exit {proc.returncode}): {tail[0][:200]}")
    pre_ms = float(rows[0][2])
    dec = {int(r[1]): float(r[4]) for r in rows[1:]}
    ms = dec[args.batch]
    mean_ctx = start + warmup + steps / 2.0
    step_bytes = weight_bytes_per_step(cfg, args.layers) + args.batch * mean_ctx * kv_bytes_per_token(cfg, args.layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(cfg, args.layers, PROMPT_LEN)
    value = args.batch * 1000.0 / ms
    line = {
        "metric": "decode_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": "qwen2-1.5b-class", "layers": args.layers, "layers_full": MODEL_1P5B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "mean_context_timed": round(mean_ctx, 1),
                   "page_size": PAGE_SIZE, "weights": "random N(0,0.02)", "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights 3.1 GB per step)", "peaks": pk["source"],
                   "build": "nv-gpu + flashinfer, sm_100a", "timing": "host clock around device_synchronize"},
        "clocks": clocks.summary(),
        # the reference's step always takes its token ids from the host and reads every request's token back
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "ms_per_step": round(ms, 4),
                "h2d_bytes_per_step": 12 * args.batch, "d2h_bytes_per_step": 8 * args.batch},
        "gpu_launches": None,
        "prefill": {"value": round(PROMPT_LEN / pre_ms * 1000.0, 1), "tokens": PROMPT_LEN, "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {f"decode_b{b}": round(b * 1000.0 / dec[b], 1) for b in pts},
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=MODEL_1P5B["num_hidden_layers"],
                    help="fewer layers than the model has (same layer sizes), where memory or time needs it")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured")
        return 2
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    if steps + warmup + 2 > CONTEXT - PROMPT_LEN:
        print(f"bench.py: --steps {steps} + --warmup {warmup} do not fit between the prompt and the context limit")
        return 2

    import torch
    from zedinfer_b200.csrc import build
    from zedinfer_b200.engine.core import EngineCore
    build.compile_all(EngineCore.kernel_libraries("bfloat16") + ["gemm_tcgen05", "attention_tcgen05"], verbose=False)
    cfg = dict(MODEL_1P5B, num_hidden_layers=args.layers)
    pk = peaks()
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    core = EngineCore(None, "bfloat16", config=cfg, random_seed=SEED, page_size=PAGE_SIZE,
                      max_tokens=max_batch * CONTEXT, max_requests=max_batch, max_seq_len=CONTEXT,
                      cuda_graphs=True)             # the engine's default: recurring steps are replayed as graphs

    clocks = ClockSampler()
    clocks.start()
    prefill = measure_prefill(core, cfg, args.layers, warmup=3, reps=5, pk=pk)
    dev = measure_decode_device(core, cfg, args.batch, steps, warmup)
    e2e = measure_decode_e2e(core, cfg, args.batch, steps, warmup)
    e2e_sync = measure_decode_e2e(core, cfg, args.batch, steps, warmup, run_ahead=False)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(measure_decode_device(core, cfg, b, min(steps, 128), warmup)["tok_s"], 1)
    head_ms = measure_head(core, cfg, args.batch)
    clocks.stop()
    core.check_kernels()            # a bounded wait that ran out inside a kernel would make the numbers void

    step_bytes = weight_bytes_per_step(cfg, args.layers) + args.batch * dev["mean_ctx"] * kv_bytes_per_token(cfg, args.layers)
    achieved = step_bytes / (dev["ms"] * 1e-3) / 1e9
    head_bytes = 2 * cfg["vocab_size"] * cfg["hidden_size"]
    layers_achieved = (step_bytes - head_bytes) / (max(dev["ms"] - head_ms, 1e-6) * 1e-3) / 1e9
    line = {
        "metric": "decode_tokens_per_s", "value": round(dev["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": round(dev["ms"], 4), "spread": dev["spread"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "qwen2-1.5b-class", "layers": args.layers, "layers_full": MODEL_1P5B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
                   "mean_context_timed": round(dev["mean_ctx"], 1), "page_size": PAGE_SIZE,
                   "weights": f"random N(0,0.02) seed {SEED}", "parallelism": "single-gpu",
                   "l2": "inputs larger than L2 (weights 3.1 GB per step)", "peaks": pk["source"]},
        "clocks": clocks.summary(),
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms"], 4),
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"], "spread": e2e["spread"],
                "host_in_step": {"value": round(e2e_sync["tok_s"], 1), "ms_per_step": round(e2e_sync["ms"], 4),
                                 "h2d_bytes_per_step": e2e_sync["h2d"]}},
        "gpu_launches": dev["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4),
                     "without_head": {"head_ms": round(head_ms, 4), "achieved": round(layers_achieved, 1),
                                      "frac": round(layers_achieved / pk["hbm_gbs"], 4)}},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
