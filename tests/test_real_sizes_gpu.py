"""The engine against the plain implementation at the layer sizes of the 1.5B-class benchmark model: hidden 1,536,
12 query heads over 2 key/value heads of 128, intermediate 8,960, vocabulary 151,936, untied head, 2 of its 28
layers (depth repeats the same kernels; width is what the tiny models cannot show).  The weights are drawn, not
stored: the engine draws them on the GPU from (seed 3, tensor name, element index), the plain implementation draws
them on the CPU with its own restatement of that rule, and the two must hold the same bits before any logit is
compared.  Requests of a few hundred tokens go through the four ways of cutting the work, in float32 and bfloat16.
"""
import random

import pytest
import torch

import traces
from plain import qwen2_plain as P
from replay_util import first_bad, first_bad_wanted, run_trace

pytestmark = pytest.mark.gpu

LAYERS, OF_LAYERS = 2, 28
REAL = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": LAYERS, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 8960, "vocab_size": 151936, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 4096,
}
SEED = 3
# Absolute, on logits whose largest magnitude is about 4 here (weights N(0, 0.02), width 1,536): the same figures as
# the tiny models' tests use on logits of magnitude 3.
TOL = {"float32": 2e-4, "bfloat16": 6e-2}
LENGTHS = [260, 150, 330]
EXTRA = [64, 100]                 # the mixed family's later requests, which take the pages of finished ones


def make_requests(lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(REAL["vocab_size"]) for _ in range(n)] for i, n in enumerate(lengths)}


@pytest.fixture(scope="module")
def plain_model():
    cfg = P.config_from_dict(REAL)
    drawn = P.random_weights(cfg, SEED, device="cuda:0")      # integer arithmetic: the same bits as on the CPU, in a second
    return cfg, {"float32": drawn, "bfloat16": {k: P.round_to(v, torch.bfloat16) for k, v in drawn.items()}}


@pytest.fixture(scope="module")
def expected(plain_model):
    cfg, weights = plain_model
    requests = make_requests(LENGTHS + EXTRA, seed=17)
    out = {}
    for dtype, act in (("float32", None), ("bfloat16", torch.bfloat16)):
        out[dtype] = {rid: P.forward(cfg, weights[dtype], toks, act) for rid, toks in requests.items()}
    return requests, out


def test_the_engine_and_the_plain_implementation_draw_the_same_weights(plain_model):
    """Device, host and the plain restatement of the rule agree bit for bit, tensor by tensor."""
    from zedinfer_b200.engine.model import Model
    from zedinfer_b200.config.registry import resolve_architecture
    from zedinfer_b200.weights.random_init import draw_tensor, unit_normal
    cfg, weights = plain_model
    arch = resolve_architecture(REAL)
    specs = Model(arch.build_spec(arch.parse(dict(REAL)))).tensor_specs()
    assert set(specs) == set(weights["float32"])
    for name in ("lm_head.weight", "embed_tokens.weight", "norm.weight", "layers.1.mlp.down_proj.weight",
                 "layers.0.self_attn.k_proj.bias", "layers.1.input_layernorm.weight"):
        on_gpu = draw_tensor(SEED, name, specs[name], torch.float32, "cuda:0").cpu()
        assert torch.equal(on_gpu, weights["float32"][name]), name
        assert torch.equal(draw_tensor(SEED, name, specs[name], torch.bfloat16, "cuda:0").float().cpu(), weights["bfloat16"][name]), name
    a = unit_normal(SEED, "layers.0.mlp.up_proj.weight", 100_000, "cuda:0", first=5_000_000).cpu()
    b = unit_normal(SEED, "layers.0.mlp.up_proj.weight", 100_000, "cpu", first=5_000_000)
    assert torch.equal(a, b)
    on_cpu = P.random_values(SEED, "lm_head.weight", (2000, 1536), 0.02)            # the plain rule on the host
    assert torch.equal(on_cpu, weights["float32"]["lm_head.weight"][:2000])
    x = weights["float32"]["layers.0.mlp.gate_proj.weight"]
    assert abs(float(x.mean())) < 1e-4 and abs(float(x.std()) - 0.02) < 2e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["whole", "tail", "chunks", "mixed"])
def test_cuts_match_plain_at_benchmark_layer_sizes(expected, family, dtype):
    from zedinfer_b200.engine.core import EngineCore
    all_requests, exp = expected
    names = [f"r{i}" for i in range(len(LENGTHS) + (len(EXTRA) if family == "mixed" else 0))]
    requests = {rid: all_requests[rid] for rid in names}
    steps = {"whole": traces.whole, "tail": traces.tail_decode, "chunks": traces.chunks,
             "mixed": traces.mixed}[family](requests)
    need = traces.max_live_tokens(steps, round_to=16)
    core = EngineCore(None, dtype, config=dict(REAL), random_seed=SEED, page_size=16, num_pages=need // 16, max_requests=4)
    assert core.spec.vocab_size == 151936 and len(core.spec.layers) == LAYERS < OF_LAYERS
    got = run_trace(core, steps)
    core.check_kernels()
    bad = first_bad(got, exp[dtype], requests, TOL[dtype])
    assert bad is None, f"first wrong position {bad}"
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("graphs", [False, True])
def test_twelve_decoding_requests_at_benchmark_layer_sizes(plain_model, graphs):
    """Decode-only steps of 9 to 12 rows at full width in bfloat16: the two-tile form of the weight-streaming product
    where the weight is small enough (down, output, q/k/v with rotation and append, gate/up with the activation), the
    library for the head; a prompt portion beside them."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, weights = plain_model
    rng = random.Random(5)
    requests = make_requests([rng.randint(30, 70) for _ in range(15)], seed=23)
    steps = traces.decode_heavy(requests, seed=9, max_live=12, tail=(6, 14))
    assert max(len(st["entries"]) for st in steps if all(len(e["tokens"]) == 1 for e in st["entries"])) > 8
    need = traces.max_live_tokens(steps, round_to=16)
    core = EngineCore(None, "bfloat16", config=dict(REAL), random_seed=SEED, page_size=16, num_pages=need // 16,
                      max_requests=16, cuda_graphs=graphs)
    core.GPU_BOUND_RATIO = float("inf")
    got = run_trace(core, steps)
    core.check_kernels()
    exp = {rid: P.forward(cfg, weights["bfloat16"], toks, torch.bfloat16) for rid, toks in requests.items()}
    bad = first_bad_wanted(got, exp, TOL["bfloat16"])
    assert bad is None, f"first wrong position {bad}"


# ---- the 7B-class layer sizes -----------------------------------------------------------------------------------
LARGE = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4,
    "head_dim": 128, "intermediate_size": 18944, "vocab_size": 152064, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 4096,
}


# Weights of 0.65 x N(0, 0.02): the logits then have the magnitude of the 1.5B-class test's (largest about 4), which the
# absolute tolerances are made for; at the full scale they are 1.5 times as large, and so is what bfloat16 adds.
LARGE_INIT_SCALE = 0.65


@pytest.fixture(scope="module")
def plain_large():
    cfg = P.config_from_dict(LARGE)
    drawn = P.random_weights(cfg, SEED, init_scale=LARGE_INIT_SCALE, device="cuda:0")
    return cfg, {k: P.round_to(v, torch.bfloat16) for k, v in drawn.items()}


def test_forty_decoding_requests_at_benchmark_layer_sizes(plain_model, monkeypatch):
    """Decode-only steps of 17 to 40 rows at the 1.5B-class sizes, bfloat16, captured: the library's products, the
    rotation and the activation as kernels of their own, and the down product as a batched product over four ranges of
    K whose float32 sums the next norm adds (the last layer's by the final norm, at the wanted rows only)."""
    from zedinfer_b200 import ops
    from zedinfer_b200.engine.core import EngineCore
    cfg, weights = plain_model
    rng = random.Random(11)
    requests = {f"p{i}": [rng.randrange(REAL["vocab_size"]) for _ in range(rng.randint(50, 80))] for i in range(44)}
    steps = traces.decode_heavy(requests, seed=6, max_live=40, tail=(34, 46))
    need = traces.max_live_tokens(steps, round_to=16)
    core = EngineCore(None, "bfloat16", config=dict(REAL), random_seed=SEED, page_size=16, num_pages=need // 16,
                      max_requests=64, cuda_graphs=True)
    core.GPU_BOUND_RATIO = float("inf")
    part_rows = set()
    real = ops.linear_for_residual

    def counted(x, w, bias):
        y = real(x, w, bias)
        if y.dim() == 3:
            part_rows.add(x.shape[0])
        return y

    monkeypatch.setattr(ops, "linear_for_residual", counted)
    got = run_trace(core, steps)
    core.check_kernels()
    exp = {rid: P.forward(cfg, weights["bfloat16"], toks, torch.bfloat16) for rid, toks in requests.items()}
    bad = first_bad_wanted(got, exp, TOL["bfloat16"])
    assert bad is None, f"first wrong position {bad}"
    assert part_rows and min(part_rows) >= ops.RESIDUAL_PARTS_MIN_ROWS


@pytest.mark.parametrize("graphs", [False, True])
def test_forty_decoding_requests_at_7b_class_layer_sizes(plain_large, graphs, monkeypatch):
    """Hidden 3,584, 28 query heads over 4 key/value heads, intermediate 18,944, 2 of 28 layers, bfloat16.  Decode-only
    steps of up to 40 rows: the stacked gate/up weight has 136 M elements, so from 32 rows it goes to the tcgen05
    kernel with the activation in its epilogue (for smaller weights that starts at 128 rows), below that to the
    library and the separate kernel, up to 8 rows to the weight-streaming kernel with K cut in two for the narrow
    outputs; prompt portions of 64 rows beside the decoding rows."""
    from zedinfer_b200 import ops
    from zedinfer_b200.engine.core import EngineCore
    cfg, weights = plain_large
    assert 2 * LARGE["intermediate_size"] * LARGE["hidden_size"] >= ops.TC_FUSED_LARGE_ELEMENTS
    rng = random.Random(7)
    requests = {f"q{i}": [rng.randrange(LARGE["vocab_size"]) for _ in range(rng.randint(50, 80))] for i in range(44)}
    steps = traces.decode_heavy(requests, seed=4, max_live=40, tail=(34, 46))
    sizes = {len(st["entries"]) for st in steps if all(len(e["tokens"]) == 1 for e in st["entries"])}
    assert max(sizes) >= 32 and min(sizes) <= 8
    need = traces.max_live_tokens(steps, round_to=16)
    core = EngineCore(None, "bfloat16", config=dict(LARGE), random_seed=SEED, init_scale=LARGE_INIT_SCALE, page_size=16,
                      num_pages=need // 16, max_requests=64, cuda_graphs=graphs)
    core.GPU_BOUND_RATIO = float("inf")
    fused_rows = set()
    real = ops.gemm_tcgen05_tiles

    def counted(x, *a, **k):
        fused_rows.add(x.shape[0])
        return real(x, *a, **k)

    monkeypatch.setattr(ops, "gemm_tcgen05_tiles", counted)
    got = run_trace(core, steps)
    core.check_kernels()
    exp = {rid: P.forward(cfg, weights, toks, torch.bfloat16) for rid, toks in requests.items()}
    bad = first_bad_wanted(got, exp, TOL["bfloat16"])
    assert bad is None, f"first wrong position {bad}"
    assert fused_rows and min(fused_rows) >= 32 and any(r < 128 for r in fused_rows)      # the fused kernel took few rows too
