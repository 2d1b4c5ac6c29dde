"""Generation through the Python entry point and bin/trace_run as a user runs it."""
import json
import os
import random
import struct
import subprocess
import sys

import numpy as np
import pytest
import torch

import tiny
import traces
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen_models")
    return {name: tiny.make_model_dir(root, name) for name in tiny.CONFIGS}


def plain_greedy(model_dir, prompt, n_new, act=None):
    cfg, w = P.load(model_dir)
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = P.greedy(P.forward(cfg, w, seq, act)[-1])
        out.append(tok)
        seq.append(tok)
    return out


@pytest.mark.parametrize("name,graphs", [("A", False), ("B", True), ("C", False), ("D", True)])
def test_greedy_generation_float32_equals_plain(models, name, graphs):
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    cfg, _ = tiny.CONFIGS[name]
    rng = random.Random(3)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (7, 13, 1)]
    engine = InferenceEngine.create(models[name], SchedulerConfig(num_kv_pages=40, kv_block_size=4, max_batch_requests=4,
                                                                  max_prefill_tokens=5, cuda_graphs=graphs),
                                    dtype="float32")
    results = engine.generate_batch(prompts, GenerationConfig(max_new_tokens=8, ignore_eos=True))
    for p, r in zip(prompts, results):
        assert r.finish_reason == "length"
        assert r.output_ids == plain_greedy(models[name], p, 8)
    assert engine.cache_stats()["live_requests"] == 0
    assert engine.cache_stats()["free_pages"] == [40] * engine.cache_stats()["groups"]


@pytest.mark.parametrize("graphs", [False, True])
def test_generation_with_a_windowed_pool_smaller_than_the_prompts(models, graphs):
    """Configuration C has a window of 24 on its upper layers.  With a token budget of 8 a step, those layers' pool is
    what three requests can hold (window + budget each), fewer pages than the three prompts have together; the prompts go
    through in portions, pages come back behind the window, and the tokens are those of the plain implementation."""
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    cfg, _ = tiny.CONFIGS["C"]
    rng = random.Random(4)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (90, 61, 33)]
    engine = InferenceEngine.create(models["C"], SchedulerConfig(num_kv_pages=80, kv_block_size=4, max_batch_requests=3,
                                                                  max_batch_tokens=8, max_prefill_tokens=8, cuda_graphs=graphs),
                                    dtype="float32")
    per_request = (24 + 8 + 2) // 4 + 1
    assert sorted(engine.cache_stats()["pages_per_group"]) == [3 * per_request, 80] and 3 * per_request < sum(-(-len(p) // 4) for p in prompts)
    results = engine.generate_batch(prompts, GenerationConfig(max_new_tokens=6, ignore_eos=True))
    for p, r in zip(prompts, results):
        assert r.finish_reason == "length" and r.output_ids == plain_greedy(models["C"], p, 6)
    st = engine.cache_stats()
    assert st["live_requests"] == 0 and sorted(st["free_pages"]) == [3 * per_request, 80] and st["preemptions"] == 0
    with pytest.raises(ValueError, match="max_step_tokens"):
        from zedinfer_b200.engine.core import StepEntry
        engine.core.step([StepEntry("too many at once", list(range(9)), [])])
    ms_prompt, ms_decode = engine.profile(40, 4)            # the measuring call cuts its prompt to the bound as well
    assert ms_prompt > 0 and ms_decode > 0 and engine.cache_stats()["live_requests"] == 0


def test_single_request_and_first_tokens(models):
    """One-token prompts and the first positions of a sequence: nothing before them in the cache."""
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    engine = InferenceEngine.create(models["B"], SchedulerConfig(num_kv_pages=16, kv_block_size=8), dtype="float32")
    for prompt in ([0], [999], [5, 6]):
        r = engine.generate_tokens(prompt, GenerationConfig(max_new_tokens=3, ignore_eos=True))
        assert r.output_ids == plain_greedy(models["B"], prompt, 3)
        assert r.stats.prompt_tokens == len(prompt) and r.stats.generated_tokens == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_stays_on_the_plain_path(models, dtype):
    """Several hundred decoded tokens, fed one by one, each compared with the whole-sequence logits: a fault
    that builds up over a long decode, or at a page's edge far from the start, shows here."""
    from zedinfer_b200.engine.core import EngineCore, StepEntry
    cfg, _ = tiny.CONFIGS["D"]
    rng = random.Random(8)
    toks = [rng.randrange(cfg["vocab_size"]) for _ in range(700)]
    pcfg, w = P.load(models["D"])
    ref = P.forward(pcfg, w, toks, torch.bfloat16 if dtype == "bfloat16" else None)
    for graphs in (False, True):
        core = EngineCore(models["D"], dtype, page_size=16, num_pages=44, max_requests=2, cuda_graphs=graphs)
        got = [core.step([StepEntry("x", toks[:100], list(range(100)))]).cpu()]
        for i in range(100, 700):
            got.append(core.step([StepEntry("x", [toks[i]], [0])]).cpu().clone())
        got = torch.cat(got)
        err = (got - ref).abs().amax(dim=1)
        tol = 3e-4 if dtype == "float32" else 8e-2
        bad = torch.nonzero(err > tol)
        assert bad.numel() == 0, f"first wrong position {int(bad[0])}, error {float(err[bad[0]])} (graphs={graphs})"
        core.end("x")


def test_temperature_sampling_is_deterministic_per_seed(models):
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    from zedinfer_b200.sampling import uniform_for
    engine = InferenceEngine.create(models["B"], SchedulerConfig(num_kv_pages=64, kv_block_size=8, max_prefill_tokens=5),
                                    dtype="float32")
    prompts = [[1], list(range(10, 27)), list(range(100, 140))]
    gc = GenerationConfig(max_new_tokens=6, use_argmax=False, temperature=0.7, seed=2, ignore_eos=True)
    together = [r.output_ids for r in engine.generate_batch(prompts, gc)]
    alone = [engine.generate_tokens(p, gc).output_ids for p in prompts]
    assert together == alone                      # a draw does not depend on who else is in the batch
    other = [r.output_ids for r in engine.generate_batch(prompts, GenerationConfig(
        max_new_tokens=6, use_argmax=False, temperature=0.7, seed=3, ignore_eos=True))]
    assert other != together
    # each token is the plain implementation's pick for the same uniform number
    cfg, w = P.load(models["B"])
    seq = list(prompts[1])
    for i, tok in enumerate(alone[1]):
        dist = P.sampling_distribution(P.forward(cfg, w, seq)[-1], 0.7, 0, 1.0)
        u = uniform_for(2, i)
        cum = torch.cumsum(dist.double(), 0)
        lo, hi = float(cum[tok] - dist[tok].double()), float(cum[tok])
        assert lo - 1e-4 <= u <= hi + 1e-4
        seq.append(tok)


def test_repetition_penalty_from_the_table_of_generated_tokens(models):
    """Requests with a repetition penalty are sampled inside the captured step, run ahead of the host, from a table
    on the device of what each has generated.  Same tokens as with the host in step and no graphs, also when pages
    run out and the youngest request is taken off the GPU and comes back (its table is built anew); and each token
    is the plain implementation's pick from the penalised logits."""
    from zedinfer_b200 import GenerationConfig, InferenceRequest, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    from zedinfer_b200.sampling import uniform_for
    prompts = [list(range(1, 8)), list(range(20, 33)), [5], list(range(40, 49))]
    configs = [GenerationConfig(max_new_tokens=30, use_argmax=False, temperature=0.9, repetition_penalty=1.8, seed=3, ignore_eos=True),
               GenerationConfig(max_new_tokens=36, use_argmax=False, temperature=0.8, top_k=6, repetition_penalty=1.3, seed=7, ignore_eos=True),
               GenerationConfig(max_new_tokens=25, ignore_eos=True),
               GenerationConfig(max_new_tokens=33, use_argmax=False, temperature=1.1, top_p=0.9, repetition_penalty=0.7, seed=9, ignore_eos=True)]

    def run(ahead, graphs, pages):
        engine = InferenceEngine.create(models["A"], SchedulerConfig(num_kv_pages=pages, kv_block_size=4, max_batch_requests=4,
                                                                     run_ahead=ahead, cuda_graphs=graphs), dtype="float32")
        futures = [engine.submit_async(InferenceRequest(p, c)) for p, c in zip(prompts, configs)]
        engine.run_loop()
        assert engine.cache_stats()["live_requests"] == 0
        return [f.result() for f in futures], engine

    base, e0 = run(False, False, 64)
    assert e0.steps_run_ahead == 0 and all(r.error is None for r in base)
    for pages in (64, 24):                 # 24 pages: the youngest request is preempted in mid-decode
        got, e1 = run(True, True, pages)
        assert e1.steps_run_ahead > 10
        assert any(key[1] == "sample" for key in e1.core._decode_graphs)
        if pages == 24:
            assert e1.cache_stats()["preemptions"] > 0
        for a, b in zip(base, got):
            assert a.output_ids == b.output_ids and a.finish_reason == b.finish_reason
    # a small top-k and a strong penalty: the same token seldom comes twice in a row
    cfg, w = P.load(models["A"])
    seq = list(prompts[1])
    out = base[1].output_ids
    for i, tok in enumerate(out):
        dist = P.sampling_distribution(P.forward(cfg, w, seq)[-1], 0.8, 6, 1.0, recent=out[:i], repetition_penalty=1.3)
        u = uniform_for(7, i)
        cum = torch.cumsum(dist.double(), 0)
        lo, hi = float(cum[tok] - dist[tok].double()), float(cum[tok])
        assert dist[tok] > 0 and lo - 1e-4 <= u <= hi + 1e-4, (i, tok)
        seq.append(tok)


def test_top_k_one_is_greedy_and_stop_token_ends(models):
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    engine = InferenceEngine.create(models["A"], SchedulerConfig(num_kv_pages=32, kv_block_size=4), dtype="float32")
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    greedy = plain_greedy(models["A"], prompt, 6)
    r = engine.generate_tokens(prompt, GenerationConfig(max_new_tokens=6, use_argmax=False, temperature=1.5, top_k=1,
                                                        seed=5, ignore_eos=True))
    assert r.output_ids == greedy
    engine.scheduler.stop_token_ids = frozenset([greedy[2]])
    r = engine.generate_tokens(prompt, GenerationConfig(max_new_tokens=6))
    first = greedy.index(greedy[2])
    assert r.finish_reason == "stop" and r.output_ids == greedy[:first + 1], (r.finish_reason, r.error, r.output_ids)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_of_the_host_changes_no_token(models, dtype):
    """Steady decode launches the next step before the host has read this one's tokens.  Same tokens as with the
    host in step, with greedy and with sampled requests side by side, with requests of different lengths (one ends
    early, one by a stop token while a step with its row is already in flight) and with pages that run out."""
    from zedinfer_b200 import GenerationConfig, InferenceRequest, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    prompts = [list(range(1, 8)), list(range(20, 33)), [5], list(range(40, 49))]
    configs = [GenerationConfig(max_new_tokens=40, ignore_eos=True),
               GenerationConfig(max_new_tokens=11, use_argmax=False, temperature=0.8, top_k=20, seed=7, ignore_eos=True),
               GenerationConfig(max_new_tokens=25),                               # stops at the stop token set below
               GenerationConfig(max_new_tokens=33, use_argmax=False, temperature=1.1, top_p=0.9, seed=9, ignore_eos=True)]

    def run(ahead, pages):
        engine = InferenceEngine.create(models["A"], SchedulerConfig(num_kv_pages=pages, kv_block_size=4, max_batch_requests=4,
                                                                     run_ahead=ahead), dtype=dtype)
        stop = plain_greedy(models["A"], prompts[2], 9)[8] if dtype == "float32" else None
        if stop is not None:
            engine.scheduler.stop_token_ids = frozenset([stop])
        futures = [engine.submit_async(InferenceRequest(p, c)) for p, c in zip(prompts, configs)]
        engine.run_loop()
        assert engine.cache_stats()["live_requests"] == 0
        assert engine.cache_stats()["free_pages"] == [pages] * engine.cache_stats()["groups"]
        return [f.result() for f in futures], engine

    base, e0 = run(False, 64)
    assert e0.steps_run_ahead == 0
    for pages in (64, 24):                 # 24 pages: the youngest request is preempted in mid-decode
        got, e1 = run(True, pages)
        assert e1.steps_run_ahead > 10
        for a, b in zip(base, got):
            assert a.output_ids == b.output_ids and a.finish_reason == b.finish_reason
    if dtype == "float32":
        assert base[2].finish_reason == "stop" and len(base[2].output_ids) <= 9
        assert base[0].output_ids == plain_greedy(models["A"], prompts[0], 40)


def test_preemption_recomputes_and_gives_the_same_tokens(models):
    """So few pages that the youngest request is taken off the GPU in mid-decode and recomputed later."""
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    prompts = [list(range(1, 8)), list(range(20, 28))]
    engine = InferenceEngine.create(models["A"], SchedulerConfig(num_kv_pages=6, kv_block_size=4, on_exhaust="preempt"),
                                    dtype="float32")
    results = engine.generate_batch(prompts, GenerationConfig(max_new_tokens=9, ignore_eos=True))
    assert engine.scheduler.num_preemptions >= 1
    for p, r in zip(prompts, results):
        assert r.finish_reason == "length" and r.output_ids == plain_greedy(models["A"], p, 9)
    engine = InferenceEngine.create(models["A"], SchedulerConfig(num_kv_pages=6, kv_block_size=4, on_exhaust="fail"),
                                    dtype="float32")
    results = engine.generate_batch(prompts, GenerationConfig(max_new_tokens=9, ignore_eos=True))
    assert sorted(r.finish_reason for r in results) == ["error", "length"]
    assert "KV cache exhausted during decode" in [r for r in results if r.error][0].error


def test_fails_loudly_without_a_gpu_tensor_or_a_known_architecture(models, tmp_path):
    from zedinfer_b200.config import ConfigError
    from zedinfer_b200.engine.core import EngineCore
    with pytest.raises(RuntimeError, match="GPU only"):
        EngineCore(models["A"], "float32", device="cpu")
    bad = tmp_path / "other"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps(dict(tiny.TINY_A, architectures=["MambaForCausalLM"], model_type="mamba")))
    with pytest.raises(ConfigError, match="Unsupported model"):
        EngineCore(str(bad), "float32")


# ---- bin/trace_run, as a separate program ----------------------------------------------------------------
def run_trace_program(model_dir, dtype, steps, out_dir, max_tokens):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for st in steps:                              # the next step goes in only after "done <step>" came back
        proc.stdin.write(json.dumps(st) + "\n")
        proc.stdin.flush()
        line = proc.stdout.readline().strip()
        assert line == f"done {st['step']}", line
    proc.stdin.close()
    assert proc.wait(timeout=60) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    cfg, _ = tiny.CONFIGS["B"]
    rng = random.Random(21)
    requests = {f"q{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate([40, 64, 90, 17, 70, 33])}
    steps = traces.mixed(requests, seed=4)
    steps[3]["entries"][0]["want"] = []           # a step may want nothing of a request
    need = traces.max_live_tokens(steps, round_to=64)
    out = tmp_path / f"out_{dtype}"
    run_trace_program(models["B"], dtype, steps, out, need)
    pcfg, w = P.load(models["B"])
    act = torch.bfloat16 if dtype == "bfloat16" else None
    ref = {rid: P.forward(pcfg, w, toks, act) for rid, toks in requests.items()}
    progress = {}
    worst = 0.0
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        path = out / f"{st['step']}.f32"
        if wanted == 0:
            assert not path.exists()
        else:
            arr = np.fromfile(path, dtype="<f4").reshape(wanted, cfg["vocab_size"])
        row = 0
        for e in st["entries"]:
            base = progress.get(e["id"], 0)
            for j in e["want"]:
                worst = max(worst, float(np.abs(arr[row] - ref[e["id"]][base + j].numpy()).max()))
                row += 1
            progress[e["id"]] = base + len(e["tokens"])
    assert worst < (2e-4 if dtype == "float32" else 6e-2), worst


# ---- the command-line programs -------------------------------------------------------------------------
def test_ping_prints_the_plain_greedy_tokens(models, capsys):
    from zedinfer_b200.cli import ping
    cfg, _ = tiny.CONFIGS["B"]
    prompt = [3, 141, 59, 26, 535, 89, 79]
    rc = ping.main([models["B"], "--dtype", "float32", "--prompt", " ".join(map(str, prompt)), "--max-new-tokens", "6",
                    "--kv-pages", "16", "--kv-block-size", "8"])
    assert rc == 0
    printed = capsys.readouterr().out.strip().splitlines()[-1]
    assert [int(t) for t in printed.split()] == plain_greedy(models["B"], prompt, 6)


def test_bench_programs_run_from_a_bare_config_with_weights_drawn_on_the_device(tmp_path, capsys):
    """--random-weights: the model path is a config.json alone; batch_bench draws prompt lengths from a range and
    reports steps, first-token times and preemptions."""
    from zedinfer_b200.cli import batch_bench, bench
    cfg, _ = tiny.CONFIGS["D"]
    path = tmp_path / "config.json"
    path.write_text(json.dumps(cfg))
    common = [str(path), "--random-weights", "7", "--kv-pages", "40", "--max-seq-len", "128"]
    assert bench.main(common + ["-p", "24", "-d", "5", "-r", "1"]) == 0
    out = capsys.readouterr().out
    assert "Prefill:" in out and "Decode :" in out
    assert batch_bench.main(common + ["-b", "5", "-p", "6", "--prefill-len-max", "40", "-d", "7", "-r", "1",
                                      "--warmup-rounds", "1", "--max-prefill-tokens", "16"]) == 0
    out = capsys.readouterr().out
    assert "5 requests, 35 tokens generated" in out and "Preemptions" in out and "First token" in out


def test_consistency_program_finds_float32_bit_equal_however_it_is_cut(tmp_path, capsys):
    """bin/zedinfer-consistency on a tiny configuration: whole, tail decoded, changing portions and mixed with page
    reuse; it returns 0 only if every float32 logit is the same bit pattern in all four."""
    from zedinfer_b200.cli import consistency
    cfg, _ = tiny.CONFIGS["D"]
    path = tmp_path / "config.json"
    path.write_text(json.dumps(dict(cfg, max_position_embeddings=512)))
    assert consistency.main([str(path), "--random-weights", "5", "--tokens", "150", "--requests", "6"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert {(l["dtype"], l["mode"]) for l in lines} >= {("float32", "tail"), ("float32", "portions"), ("float32", "mixed"),
                                                        ("bfloat16", "mixed"), ("bfloat16", "whole")}
    assert all(l["values_not_bit_equal"] == 0 for l in lines if l["dtype"] == "float32")
    assert all(l["worst_abs_diff"] < 6e-2 for l in lines if l["dtype"] == "bfloat16")


def test_a_capture_survives_the_collection_of_an_engine_that_is_gone(models):
    """An engine that was dropped leaves its CUDA graphs in reference cycles; if Python's collector destroys them in
    the middle of another engine's capture, that capture is lost ("operation not permitted when stream is
    capturing").  Captures therefore collect before they start.  Here the old engine's graphs are kept from the
    collector until the new engine captures, and a collection is forced inside every captured forward pass."""
    import gc
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    gc.collect()
    gc.disable()
    try:
        e1 = InferenceEngine.create(models["A"], SchedulerConfig(num_kv_pages=32, kv_block_size=4), dtype="float32")
        for _ in range(2):
            assert e1.generate_tokens(prompt, GenerationConfig(max_new_tokens=5, ignore_eos=True)).error is None
        assert e1.core._decode_graphs
        del e1                                     # its graphs stay behind, uncollected
        e2 = InferenceEngine.create(models["A"], SchedulerConfig(num_kv_pages=32, kv_block_size=4), dtype="float32")
        e2.core.GPU_BOUND_RATIO = float("inf")     # the prompt's step is captured at its second appearance
        forward = e2.core.model.forward

        def forward_with_a_collection(*args, **kw):
            if torch.cuda.is_current_stream_capturing():
                gc.collect()
            return forward(*args, **kw)
        e2.core.model.forward = forward_with_a_collection
        for _ in range(3):
            r = e2.generate_tokens(prompt, GenerationConfig(max_new_tokens=5, ignore_eos=True))
            assert r.error is None and r.finish_reason == "length", (r.finish_reason, r.error)
        assert e2.core._step_graphs
    finally:
        gc.enable()


def test_generation_across_the_length_where_the_decode_graph_changes(tmp_path):
    """Requests that decode from below to above the context length from which the captured decode step plans for
    clusters that share a request: the engine, running ahead of the host, moves from one captured graph to the other
    (greedy and sampled rows), and the tokens are those of the engine without graphs."""
    from zedinfer_b200 import GenerationConfig, InferenceRequest, SchedulerConfig, ops
    from zedinfer_b200.engine import InferenceEngine
    edge = ops.decode_attention_split_from()
    cfg = dict(tiny.TINY_E, max_position_embeddings=edge + 200)
    path = tmp_path / "config.json"
    path.write_text(json.dumps(cfg))
    rng = random.Random(11)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (edge - 20, 50, edge - 33)]
    configs = [GenerationConfig(max_new_tokens=45, ignore_eos=True),
               GenerationConfig(max_new_tokens=45, ignore_eos=True),
               GenerationConfig(max_new_tokens=60, use_argmax=False, temperature=0.8, top_k=30, repetition_penalty=1.2, seed=4, ignore_eos=True)]

    def run(graphs):
        sc = SchedulerConfig(num_kv_pages=(2 * edge + 600) // 16, kv_block_size=16, max_batch_requests=4, max_prefill_tokens=2048,
                             max_batch_tokens=4096, cuda_graphs=graphs, run_ahead=graphs)
        engine = InferenceEngine.create(str(path), sc, dtype="bfloat16", random_seed=9)
        futures = [engine.submit_async(InferenceRequest(p, c)) for p, c in zip(prompts, configs)]
        engine.run_loop()
        return [f.result() for f in futures], engine

    base, _ = run(False)
    got, engine = run(True)
    assert all(r.error is None for r in base + got)
    for a, b in zip(base, got):
        assert a.output_ids == b.output_ids
    reaches = {key[2] for key in engine.core._decode_graphs}
    assert reaches == {edge - 1, edge + 200} and engine.steps_run_ahead > 20


def test_profile_step_runs_a_small_step_of_each_kind(capsys):
    """The program that stands between cudaProfilerStart and Stop for the ncu captures: every mode at a small size."""
    from zedinfer_b200.cli import profile_step
    small = ["--layers", "2", "--hidden", "256", "--heads", "4", "--kv-heads", "2", "--head-dim", "64",
             "--intermediate", "512", "--vocab", "3000", "--steps", "1"]
    for mode, more in (("decode", ["--batch", "3", "--context", "40"]), ("decode", ["--batch", "3", "--context", "40", "--graphs"]),
                       ("prefill", ["--tokens", "70"]), ("mixed", ["--batch", "2", "--context", "30", "--tokens", "50"]),
                       ("sample", ["--batch", "3"])):
        assert profile_step.main(["--mode", mode] + more + small) == 0
        line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert line["mode"] == mode and (line.get("ms_per_step", 0) > 0 or line.get("us_per_call", 0) > 0)


def test_engine_default_sampling_comes_from_generation_config_json(models, tmp_path, monkeypatch):
    """A folder whose generation_config.json says do_sample: a request without sampling options is sampled with the
    folder's values (same tokens as a request that states them), ZEDINFER_FORCE_ARGMAX brings greedy back, and a
    request that insists on greedy gets it (src/zedinfer/engine.cpp:49-126, src/zedinfer/scheduler.cpp:576-601)."""
    import shutil
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    folder = tmp_path / "with_generation_config"
    shutil.copytree(models["B"], folder)
    (folder / "generation_config.json").write_text(json.dumps(
        {"do_sample": True, "temperature": 1.4, "top_k": 30, "top_p": 0.97, "seed": 11}))
    prompt = [3, 141, 59, 26, 535, 89, 79]
    sc = SchedulerConfig(num_kv_pages=32, kv_block_size=8)
    monkeypatch.delenv("ZEDINFER_FORCE_ARGMAX", raising=False)
    engine = InferenceEngine.create(str(folder), sc, dtype="float32")
    assert not engine.default_generation.use_argmax and engine.default_generation.top_k == 30
    by_default = engine.generate_tokens(prompt, GenerationConfig(max_new_tokens=12, ignore_eos=True)).output_ids
    stated = engine.generate_tokens(prompt, GenerationConfig(max_new_tokens=12, ignore_eos=True, use_argmax=False,
                                                             temperature=1.4, top_k=30, top_p=0.97, seed=11)).output_ids
    greedy = plain_greedy(models["B"], prompt, 12)
    assert by_default == stated and by_default != greedy
    insisted = engine.generate_tokens(prompt, GenerationConfig(max_new_tokens=12, ignore_eos=True,
                                                               has_sampling_override=True)).output_ids
    assert insisted == greedy
    monkeypatch.setenv("ZEDINFER_FORCE_ARGMAX", "1")
    forced = InferenceEngine.create(str(folder), sc, dtype="float32")
    assert forced.generate_tokens(prompt, GenerationConfig(max_new_tokens=12, ignore_eos=True)).output_ids == greedy


def test_greedy_batch_chooses_inside_the_captured_step(models):
    """Five greedy requests of different lengths (a bucket of eight: three rows of padding whose positions move on
    with the others'), decoded with the choice and the hand-over inside the captured step and with steps launched
    ahead of the host: every request gets the plain implementation's tokens, and the pool is whole afterwards."""
    from zedinfer_b200 import GenerationConfig, InferenceRequest, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    cfg, _ = tiny.CONFIGS["B"]
    rng = random.Random(77)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (5, 19, 2, 33, 11)]
    news = [40, 23, 31, 9, 40]
    engine = InferenceEngine.create(models["B"], SchedulerConfig(num_kv_pages=64, kv_block_size=8, max_batch_requests=8),
                                    dtype="float32")
    futs = [engine.submit_async(InferenceRequest(p, GenerationConfig(max_new_tokens=n, ignore_eos=True)))
            for p, n in zip(prompts, news)]
    engine.run_loop()
    for p, n, f in zip(prompts, news, futs):
        r = f.result()
        assert r.error is None and r.output_ids == plain_greedy(models["B"], p, n)
    assert any(key[1] for key in engine.core._decode_graphs)
    assert engine.steps_run_ahead > 10
    engine.core.cache.check()
    assert engine.core.cache.num_live == 0
