"""The engine against the plain implementation, in float32 and in bfloat16, under every way of
cutting the work: whole prompts, a decoded tail, portions of changing size, and mixed batches with
so few pages that they are used again."""
import math
import random

import pytest
import torch

import tiny
import traces
from plain import qwen2_plain as P
from replay_util import compare, first_bad, first_bad_wanted, run_trace

pytestmark = pytest.mark.gpu

# Tolerances, absolute on logits of magnitude ~3: float32 differs from the plain implementation by the
# order of sums only; bfloat16 is compared with the plain implementation rounding its activations to
# bfloat16 at the same places, so what is left is the order of sums again, seen through bfloat16 steps.
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def make_requests(cfg, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: tiny.make_model_dir(root, name) for name in tiny.CONFIGS}


def expected_logits(model_dir, requests, dtype):
    cfg, w = P.load(model_dir)
    act = torch.bfloat16 if dtype == "bfloat16" else None
    return {rid: P.forward(cfg, w, toks, act) for rid, toks in requests.items()}


LENGTHS = {"A": [7, 13, 70, 45], "B": [1, 17, 40, 90], "C": [60, 5, 100, 33], "D": [50, 130, 9], "E": [33, 150, 80],
           "F": [150, 47, 260, 90]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("family", ["whole", "tail", "chunks", "mixed"])
def test_cuts_match_plain(models, name, dtype, family):
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = tiny.CONFIGS[name]
    requests = make_requests(cfg, LENGTHS[name] + ([64, 31, 77] if family == "mixed" else []), seed=11)
    steps = {"whole": traces.whole, "tail": traces.tail_decode, "chunks": traces.chunks,
             "mixed": traces.mixed}[family](requests)
    page = {"A": 4, "B": 8, "C": 16, "D": 16, "E": 16, "F": 16}[name]
    need = traces.max_live_tokens(steps, round_to=page)
    core = EngineCore(models[name], dtype, page_size=page, num_pages=need // page, max_requests=4)
    got = run_trace(core, steps)
    exp = expected_logits(models[name], requests, dtype)
    bad = first_bad(got, exp, requests, TOL[dtype])
    worst, where = compare(got, exp, requests)
    assert bad is None, f"first wrong position {bad}; worst {worst} at {where}"
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "F"])
@pytest.mark.parametrize("family", ["chunks", "mixed"])
def test_a_windowed_group_with_a_pool_of_its_own_size(models, name, dtype, family):
    """The engine is told the most tokens a step brings of one request; the layers with a window then share a pool
    that is only as large as four requests can fill, with a scratch page of its own number, and the logits are
    those of the plain implementation."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = tiny.CONFIGS[name]
    requests = make_requests(cfg, LENGTHS[name] + ([64, 31, 77] if family == "mixed" else []), seed=13)
    steps = {"chunks": traces.chunks, "mixed": traces.mixed}[family](requests)
    bound = max(len(e["tokens"]) for st in steps for e in st["entries"])
    window = cfg["sliding_window"]
    per_request = (window + bound + 14) // 16 + 1
    core = EngineCore(models[name], dtype, page_size=16, num_pages=8 * per_request, max_requests=4, max_step_tokens=bound)
    sizes = {g.window: g.num_pages for g in core.cache.groups}
    assert sizes == {None: 8 * per_request, window: 4 * per_request}
    assert core.cache.scratch_pages == [g.num_pages for g in core.cache.groups]
    got = run_trace(core, steps)
    bad = first_bad(got, expected_logits(models[name], requests, dtype), requests, TOL[dtype])
    assert bad is None, f"first wrong position {bad}"
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,max_live", [("D", 12), ("D", 40), ("E", 12), ("E", 40), ("F", 12)])
def test_many_decoding_requests_match_plain(models, name, max_live, dtype, graphs):
    """Steps as a scheduler makes them with many requests live: decode-only steps of up to 12 and up to 40 rows
    (9 to 16 rows: the two-tile form of the weight-streaming product; 17 and more: library products with separate
    rotation and activation kernels, decode attention with smaller clusters), one prompt portion beside up to 37
    decoding requests, requests that sit steps out, and a pool that later requests fill again.  With graphs the
    decode-only steps replay the captured buckets 16, 32 and 64 with rows of padding, and mixed steps whose counts
    come back are captured too.  Every wanted logit is the plain implementation's."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = tiny.CONFIGS[name]
    rng = random.Random(77 + max_live)
    n_req = max_live + max_live // 3
    lengths = [rng.randint(50, 110) for _ in range(n_req)]
    requests = make_requests(cfg, lengths, seed=13)
    steps = traces.decode_heavy(requests, seed=5, max_live=max_live, tail=(44, 64) if max_live > 16 else (8, 24))
    rows = [len(st["entries"]) for st in steps if all(len(e["tokens"]) == 1 for e in st["entries"])]
    assert max(rows) > (16 if max_live > 16 else 8)
    need = traces.max_live_tokens(steps, round_to=16)
    core = EngineCore(models[name], dtype, page_size=16, num_pages=need // 16, max_requests=64, cuda_graphs=graphs)
    core.GPU_BOUND_RATIO = float("inf")
    got = run_trace(core, steps)
    exp = expected_logits(models[name], requests, dtype)
    bad = first_bad_wanted(got, exp, TOL[dtype])
    assert bad is None, f"first wrong position {bad}"
    assert len(got) > sum(min(len(t) - 1, 8) for t in requests.values())
    if graphs:
        assert {g.bucket for g in core._decode_graphs.values()} >= ({16, 32, 64} if max_live > 16 else {8, 16})
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("graphs", [False, True])
def test_decoding_across_the_length_from_which_clusters_share_a_request(graphs):
    """A request decodes from below to above the context length from which the decode attention lets several
    clusters share one request's keys, a short request beside it.  With graphs the step moves from the graph captured
    for short contexts (no kernel that adds the clusters' parts) to the one captured for the longest sequence."""
    from zedinfer_b200 import ops
    from zedinfer_b200.engine.core import EngineCore
    edge = ops.decode_attention_split_from()
    cfg = dict(tiny.TINY_E, max_position_embeddings=edge + 300)
    rng = random.Random(3)
    tail = 40
    requests = {"long": [rng.randrange(cfg["vocab_size"]) for _ in range(edge + 18)],
                "short": [rng.randrange(cfg["vocab_size"]) for _ in range(90)]}
    steps = []
    for rid, toks in requests.items():
        head = len(toks) - tail
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
    for i in range(tail):
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": rid, "tokens": [toks[len(toks) - tail + i]], "want": [0]} for rid, toks in requests.items()]})
    steps[-1]["end"] = list(requests)
    need = traces.max_live_tokens(steps, round_to=16)
    scale = tiny.INIT_SCALES.get("E", tiny.INIT_SCALE)
    core = EngineCore(None, "bfloat16", config=cfg, random_seed=11, page_size=16, num_pages=need // 16, max_requests=4,
                      cuda_graphs=graphs, init_scale=scale)
    got = run_trace(core, steps)
    core.check_kernels()
    pcfg = P.config_from_dict(cfg)
    weights = {k: P.round_to(v, torch.bfloat16)
               for k, v in P.random_weights(pcfg, 11, init_scale=scale, device="cuda:0").items()}
    exp = {rid: P.forward(pcfg, weights, toks, torch.bfloat16).cpu() for rid, toks in requests.items()}
    bad = first_bad_wanted(got, exp, TOL["bfloat16"])
    assert bad is None, f"first wrong position {bad}"
    assert len(got) == 2 * tail + 2
    if graphs:
        assert {key[2] for key in core._decode_graphs} == {edge - 1, edge + 300}
    assert core.cache.num_live == 0


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "F"])
def test_float32_is_the_same_however_it_is_cut(models, name):
    """In float32 every sum has one order, so the cuts agree to the last bit."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = tiny.CONFIGS[name]
    requests = make_requests(cfg, [70, 45, 64, 31], seed=5)
    outs = []
    for fam in (traces.whole, traces.tail_decode, traces.chunks, traces.mixed):
        core = EngineCore(models[name], "float32", page_size=8, num_pages=64, max_requests=4)
        outs.append(run_trace(core, fam(requests)))
    for other in outs[1:]:
        for key, ref in outs[0].items():
            assert torch.equal(ref, other[key]), f"{key} differs between cuts"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("plain_products", [False, True])
def test_a_long_prompt_takes_the_many_row_kernels(models, dtype, plain_products, monkeypatch):
    """1,024 tokens in one step: in bfloat16 the gate/up product runs on the tcgen05 kernel for many rows (SM pairs,
    SiLU-mul epilogue), with ``ops.TC_PLAIN_PRODUCTS`` the other three products of a layer too, and the attention
    on its tcgen05 kernel with eight key tiles; the logits at the first, the last and a few positions in between
    (tile edges among them) are the plain implementation's."""
    from zedinfer_b200 import ops
    monkeypatch.setattr(ops, "TC_PLAIN_PRODUCTS", plain_products)
    from zedinfer_b200.engine.core import EngineCore, StepEntry
    cfg, _ = tiny.CONFIGS["D"]
    calls = {"tiles": 0, "attention": 0}
    real_tiles, real_attn = ops.gemm_tcgen05_tiles, ops.prefill_attention_tcgen05

    def counted_tiles(*a, **k):
        calls["tiles"] += 1
        return real_tiles(*a, **k)

    def counted_attn(*a, **k):
        calls["attention"] += 1
        return real_attn(*a, **k)

    monkeypatch.setattr(ops, "gemm_tcgen05_tiles", counted_tiles)
    monkeypatch.setattr(ops, "prefill_attention_tcgen05", counted_attn)
    rng = random.Random(21)
    toks = [rng.randrange(cfg["vocab_size"]) for _ in range(1024)]
    want = [0, 1, 127, 128, 129, 511, 640, 1000, 1023]
    core = EngineCore(models["D"], dtype, page_size=16, num_pages=64, max_requests=2)
    logits = core.step([StepEntry("long", toks, want)]).float().cpu()
    core.end("long")
    exp = expected_logits(models["D"], {"long": toks}, dtype)["long"]
    for row, p in enumerate(want):
        d = float((logits[row] - exp[p]).abs().max())
        assert d <= TOL[dtype], (p, d)
    if dtype == "bfloat16":
        assert calls["tiles"] == (4 if plain_products else 1) * cfg["num_hidden_layers"]
        assert calls["attention"] == cfg["num_hidden_layers"]
    else:
        assert calls["tiles"] == 0 and calls["attention"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_captured_steps_equal_eager_steps(models, name, dtype):
    """With graphs on, a step whose counts (tokens, segments, tiles, wanted rows) come back is captured at its
    second appearance and replayed afterwards; the logits are the eager ones to the last bit.  Portions of one
    size repeat here, alone and beside decoding requests, and pages are freed and used again in between."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = tiny.CONFIGS[name]
    requests = make_requests(cfg, [96, 96, 64, 96], seed=31)
    ids = list(requests)
    steps, k = [], 0
    # r0 in portions of 16; then r1 in portions of 16 beside decoded tokens of nobody (same counts as before);
    # then r2 and r3 in portions of 32 with r0's last tokens fed one by one beside them
    for rid in ids[:2]:
        toks = requests[rid]
        for s0 in range(0, len(toks), 16):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[s0:s0 + 16], "want": [15]}], "end": []})
            k += 1
        steps[-1]["end"] = [rid]
    a, b = requests[ids[2]], requests[ids[3]]
    for i in range(2):
        steps.append({"step": k, "entries": [{"id": ids[2], "tokens": a[32 * i:32 * i + 32], "want": [0, 31]}], "end": []})
        k += 1
    for i in range(3):
        steps.append({"step": k, "entries": [{"id": ids[2], "tokens": [a[0]], "want": [0]},
                                             {"id": ids[3], "tokens": b[32 * i:32 * i + 32], "want": [31]}], "end": []})
        k += 1
    steps[-1]["end"] = [ids[2], ids[3]]
    page = {"A": 4, "D": 16}[name]
    outs = []
    for graphs in (False, True):
        core = EngineCore(models[name], dtype, page_size=page, num_pages=256 // page + 8, max_requests=4, cuda_graphs=graphs)
        core.GPU_BOUND_RATIO = float("inf")       # capture at the second appearance, however long the GPU takes
        got = {}
        for st in steps:
            from zedinfer_b200.engine.core import StepEntry
            logits = core.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]])
            got[st["step"]] = logits.float().cpu().clone()
            for rid in st["end"]:
                core.end(rid)
        outs.append(got)
        if graphs:
            assert len(core._step_graphs) >= 3, list(core._step_graphs)
        core.cache.check()
    for key, ref in outs[0].items():
        assert torch.equal(ref, outs[1][key]), f"step {key} differs between eager and captured"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_mixed_steps_with_padding_equal_eager_steps(models, dtype):
    """Three decoding requests beside a prompt portion: the captured form pads the single tokens to four with a
    token on the scratch page; logits are the eager ones to the last bit, and the padding leaves the cache alone."""
    from zedinfer_b200.engine.core import EngineCore, StepEntry
    cfg, _ = tiny.CONFIGS["D"]
    requests = make_requests(cfg, [70, 70, 70, 128], seed=41)
    ids = list(requests)
    steps = [[(rid, requests[rid][:64], [63])] for rid in ids[:3]]
    for i in range(4):
        steps.append([(rid, [requests[rid][64 + i]], [0]) for rid in ids[:3]] +
                     [(ids[3], requests[ids[3]][32 * i:32 * i + 32], [31])])
    outs = []
    for graphs in (False, True):
        core = EngineCore(models["D"], dtype, page_size=16, num_pages=40, max_requests=4, cuda_graphs=graphs)
        core.GPU_BOUND_RATIO = float("inf")
        got = []
        for st in steps:
            got.append(core.step([StepEntry(*e) for e in st]).float().cpu().clone())
        if graphs:
            assert any(g.pad == 1 for g in core._step_graphs.values())
        for rid in ids:
            core.end(rid)
        core.cache.check()
        outs.append(got)
    for i, (a, b) in enumerate(zip(*outs)):
        assert torch.equal(a, b), f"step {i} differs between eager and captured"
    exp = expected_logits(models["D"], requests, dtype)
    last = outs[1][-1]                      # rows: r0, r1, r2 at position 67, r3 at position 127
    for row, rid in enumerate(ids[:3]):
        assert float((last[row] - exp[rid][67]).abs().max()) <= TOL[dtype]
    assert float((last[3] - exp[ids[3]][127]).abs().max()) <= TOL[dtype]


def test_a_step_shape_is_captured_only_if_the_host_is_the_slower_one(models):
    """The first appearance of a step shape is timed on both sides.  A shape whose GPU time exceeds the host's
    launch time by the ratio stays eager however often it comes back; any other is captured at its second
    appearance and replayed from the third."""
    from zedinfer_b200.engine.core import EngineCore, StepEntry
    cfg, _ = tiny.CONFIGS["D"]
    toks = make_requests(cfg, [96], seed=51)["r0"]
    for ratio, graphs_after in ((0.0, [0, 0, 0]), (float("inf"), [0, 1, 1])):
        core = EngineCore(models["D"], "bfloat16", page_size=16, num_pages=16, max_requests=2, cuda_graphs=True)
        core.GPU_BOUND_RATIO = ratio
        seen, outs = [], []
        for i in range(3):
            outs.append(core.step([StepEntry(("p", i), toks[:32], [31])]).float().cpu().clone())
            core.end(("p", i))
            seen.append(len(core._step_graphs))
        assert seen == graphs_after, (ratio, seen)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
