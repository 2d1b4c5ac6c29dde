"""Random workloads through InferenceEngine with captured steps, steps launched ahead of the host, prompts cut into
small portions, token budgets small enough that a windowed group's pool is cut to what the requests can hold, and
pools small enough for preemption: greedy requests must produce the plain implementation's tokens,
sampling requests the tokens of the same engine run step by step without graphs; no page may be lost."""
import random

import pytest

import tiny
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("soak_models")
    return {name: tiny.make_model_dir(root, name) for name in ("A", "B", "C", "D")}


def plain_greedy(loaded, prompt, n_new):
    cfg, w = loaded
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = P.greedy(P.forward(cfg, w, seq)[-1])
        out.append(tok)
        seq.append(tok)
    return out


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_workloads(models, seed):
    from zedinfer_b200 import GenerationConfig, InferenceEngine, InferenceRequest, SchedulerConfig
    rng = random.Random(seed)
    loaded = {n: P.load(models[n]) for n in models}
    preemptions = 0
    for trial in range(7):
        name = rng.choice(["A", "B", "C", "D"])      # C: a window on the upper layers, whose pool shrinks with the token budget
        cfg, _ = tiny.CONFIGS[name]
        page = rng.choice([4, 8, 16])
        n_req = rng.randrange(2, 9)
        prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randrange(1, 40))] for _ in range(n_req)]
        news = [rng.randrange(1, 30) for _ in range(n_req)]
        need = sum(-(-(len(p) + n) // page) for p, n in zip(prompts, news))
        biggest = max(-(-(len(p) + n) // page) for p, n in zip(prompts, news))
        pages = max(biggest + 1, int(need * rng.choice([0.5, 0.7, 1.2])))
        configs = []
        for n in news:
            if rng.random() < 0.5:
                configs.append(GenerationConfig(max_new_tokens=n, ignore_eos=True))
            else:
                configs.append(GenerationConfig(max_new_tokens=n, ignore_eos=True, use_argmax=False,
                                                temperature=rng.choice([0.7, 1.3]), top_k=rng.choice([0, 20]),
                                                top_p=rng.choice([1.0, 0.9]), seed=rng.randrange(1, 1000),
                                                repetition_penalty=rng.choice([1.0, 1.0, 1.3, 0.8])))
        outs = []
        for graphs in (True, False):
            sc = SchedulerConfig(num_kv_pages=pages, kv_block_size=page, max_batch_requests=8,
                                 max_prefill_tokens=rng.choice([5, 16, 64]) if graphs else 64,
                                 max_batch_tokens=rng.choice([24, 2048]) if graphs else 2048, cuda_graphs=graphs,
                                 run_ahead=graphs)
            engine = InferenceEngine.create(models[name], sc, dtype="float32")
            futs = [engine.submit_async(InferenceRequest(p, g)) for p, g in zip(prompts, configs)]
            engine.run_loop()
            outs.append([f.result() for f in futs])
            engine.core.cache.check()
            assert engine.core.cache.num_live == 0
            preemptions += engine.scheduler.num_preemptions
        for i in range(n_req):
            a, b = outs[0][i], outs[1][i]
            assert a.error is None and b.error is None, (trial, i, a.error, b.error)
            assert a.output_ids == b.output_ids, (trial, name, i, configs[i])
            if configs[i].use_argmax:
                assert a.output_ids == plain_greedy(loaded[name], prompts[i], news[i]), (trial, name, i)
    assert preemptions > 0
