"""Each part of a layer alone against its plain formula, and a toy mixer with state of its own, defined here,
registered, built into a model, loaded and stepped without a change to the framework's files."""
import json
import math
import os
import random

import pytest
import torch

from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def step_context(cache, dtype, portions, table_width=16):
    """portions: list of (request id, n_tokens).  Opens / extends the requests and builds the step's descriptor."""
    from zedinfer_b200.engine.core import PinnedStaging, StepEntry, build_step_context
    entries, rcs = [], []
    for rid, n in portions:
        rc = cache.get(rid) or cache.open(rid)
        cache.ensure(rc, rc.length + n)
        entries.append(StepEntry(rid, [0] * n, []))
        rcs.append(rc)
    ctx, _ = build_step_context(entries, rcs, cache, table_width, dtype, torch.device(DEV), 10, PinnedStaging())
    return ctx, entries, rcs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from zedinfer_b200.parts import ResidualStream, RMSNorm
    norm = RMSNorm(size=200, eps=1e-4)
    assert norm.tensor_specs()["weight"].shape == (200,)
    w = (1 + 0.1 * torch.randn(200)).to(dtype).to(DEV)
    norm.bind({"weight": w})
    h = torch.randn(5, 200, device=DEV)
    delta = torch.randn(5, 200, device=DEV).to(dtype)
    stream = ResidualStream(h.clone(), delta)
    out = torch.empty(5, 200, dtype=dtype, device=DEV)
    norm.forward_residual(stream, out)
    assert stream.delta is None and torch.equal(stream.h, h + delta.float())
    ref = P.rms_norm((h + delta.float()).cpu(), w.float().cpu(), 1e-4)
    assert torch.allclose(out.float().cpu(), ref, atol=2e-2 if dtype == torch.bfloat16 else 1e-5, rtol=1e-2)
    with pytest.raises(ValueError):
        RMSNorm(size=8, eps=0.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_mlp_part(dtype):
    from zedinfer_b200.parts import GatedMLP, StepContext
    mlp = GatedMLP(hidden_size=72, intermediate_size=200)
    specs = mlp.tensor_specs()
    assert specs["gate_proj.weight"].shape == (200, 72) and specs["down_proj.weight"].shape == (72, 200)
    t = {k: (0.2 * torch.randn(v.shape)).to(dtype).to(DEV) for k, v in specs.items()}
    mlp.bind(t)
    x = torch.randn(6, 72).to(dtype).to(DEV)
    ctx = StepContext(6, 1, dtype, torch.device(DEV), None, None, None, [], None, [0], [6], [0], [-1])
    y = mlp.forward(x, ctx)
    f = {k: v.float().cpu() for k, v in t.items()}
    xf = x.float().cpu()
    r = (lambda z: z.to(dtype).float()) if dtype == torch.bfloat16 else (lambda z: z)   # what the engine stores
    gate, up = r(P.linear(xf, f["gate_proj.weight"], None)), r(P.linear(xf, f["up_proj.weight"], None))
    ref = r(P.linear(r(P.swiglu(gate, up)), f["down_proj.weight"], None))
    # bfloat16: one unit in the last place of the stored output (2^-8 relative) for a differently ordered sum
    assert torch.allclose(y.float().cpu(), ref, atol=3e-2 if dtype == torch.bfloat16 else 1e-5, rtol=2e-2)
    with pytest.raises(ValueError, match="gelu"):
        GatedMLP(8, 8, activation="gelu")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 2, 32, None), (4, 4, 64, 9), (12, 2, 128, None)])
def test_attention_part_with_rope_over_portions(dtype, nh, nkv, hd, window):
    """The mixer alone: a prompt fed in portions (7, 2, 1, 20 tokens) gives what whole-sequence attention gives."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.config import PartSpec
    from zedinfer_b200.parts import AttentionMixer
    hidden, theta = 80, 20000.0
    mixer = AttentionMixer(hidden_size=hidden, num_heads=nh, num_kv_heads=nkv, head_dim=hd, window=window,
                           position=PartSpec("rope", {"head_dim": hd, "theta": theta}))
    specs = mixer.tensor_specs()
    assert "q_proj.bias" in specs and "o_proj.bias" not in specs
    g = torch.Generator().manual_seed(1)
    t = {k: (torch.randn(v.shape, generator=g) * 0.08).to(dtype).to(DEV) for k, v in specs.items()}
    mixer.bind(t)
    cache = CacheManager([(0, mixer.cache_need())], 4, max_requests=2)
    cache.allocate_device(16, dtype, DEV)
    view = cache.view_for_call(0)
    total = 30
    x = torch.randn(total, hidden, generator=g).to(dtype)
    got, done = [], 0
    for n in (7, 2, 1, 20):
        ctx, entries, rcs = step_context(cache, dtype, [("r", n)])
        got.append(mixer.forward(x[done:done + n].to(DEV), ctx, view, owns_cache=True).float().cpu())
        cache.commit(rcs[0], rcs[0].length + n)
        done += n
    got = torch.cat(got)
    f = {k: v.float().cpu() for k, v in t.items()}
    xf = x.float()
    r = (lambda z: z.to(dtype).float()) if dtype == torch.bfloat16 else (lambda z: z)
    q = r(P.linear(xf, f["q_proj.weight"], f["q_proj.bias"])).view(total, nh, hd)
    k = r(P.linear(xf, f["k_proj.weight"], f["k_proj.bias"])).view(total, nkv, hd)
    v = r(P.linear(xf, f["v_proj.weight"], f["v_proj.bias"])).view(total, nkv, hd)
    pos = torch.arange(total)
    a = r(P.attention(r(P.rope(q, pos, theta)), r(P.rope(k, pos, theta)), v, 1.0 / math.sqrt(hd), window))
    ref = P.linear(a.reshape(total, nh * hd), f["o_proj.weight"], None)
    # relative to the size of the outputs: float32 differs by the order of sums, bfloat16 by its 2^-8 steps
    tol = (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, float(ref.abs().max()))
    assert float((got - ref).abs().max()) < tol
    for bad in (dict(head_dim=40), dict(num_kv_heads=5), dict(window=0), dict(head_dim=512)):
        kw = dict(hidden_size=hidden, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                  position=PartSpec("rope", {"head_dim": hd, "theta": theta}))
        kw.update(bad)
        with pytest.raises(ValueError):
            AttentionMixer(**kw)


# ---- a toy architecture with a toy mixer ------------------------------------------------------------------
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from zedinfer_b200.cache import StateNeed
    from zedinfer_b200.config import (LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture,
                                      unregister_architecture)
    from zedinfer_b200.engine.core import EngineCore, StepEntry
    from zedinfer_b200.parts import Mixer, register_mixer, unregister
    from zedinfer_b200.weights import TensorSpec, write_random_model

    @register_mixer("toy_decay")
    class DecayMixer(Mixer):
        """y_t = s_t W^T with s_t = decay * s_{t-1} + x_t: a running state per request, no keys or values."""

        def __init__(self, hidden_size, decay):
            self.hidden_size, self.decay = hidden_size, decay

        def cache_need(self):
            return StateNeed((self.hidden_size,), torch.float32)

        def tensor_specs(self):
            return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"].float()

        def forward(self, x, ctx, cache, owns_cache):
            out = torch.empty_like(x)
            for start, n, slot in zip(ctx.seg_start_host, ctx.seg_len_host, ctx.slots_host):
                s = cache.tensor[slot]
                for i in range(start, start + n):
                    s.mul_(self.decay).add_(x[i].float())
                    out[i] = (s @ self.w.t()).to(x.dtype)
            return out

    def parse(raw):
        return raw

    def build_spec(raw):
        h = raw["hidden_size"]
        norm = PartSpec("rmsnorm", {"size": h, "eps": raw["eps"]})
        ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": raw["inter"]})
        attn = PartSpec("attention", {"hidden_size": h, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                      "position": PartSpec("rope", {"head_dim": 16, "theta": 10000.0})})
        toy = PartSpec("toy_decay", {"hidden_size": h, "decay": raw["decay"]})
        prefixes = {"mixer": "mixer.", "ffn": "mlp.", "norm1": "ln1.", "norm2": "ln2."}
        layers = tuple(LayerSpec("pre_norm", m, ffn, {"norm1": norm, "norm2": norm}, prefixes) for m in (toy, attn))
        # the run order names layer 0 twice (two state slots of its own) around the attention layer
        return ModelSpec("ToyForCausalLM", raw["vocab_size"], h, layers, (LayerCall(0), LayerCall(1), LayerCall(0)),
                         norm, True, raw["max_position_embeddings"])

    register_architecture("ToyForCausalLM", model_types=("toy",), parse=parse, build_spec=build_spec)
    try:
        raw = {"architectures": ["ToyForCausalLM"], "hidden_size": 48, "inter": 100, "vocab_size": 300, "eps": 1e-5,
               "decay": 0.8, "max_position_embeddings": 128}
        folder = write_random_model(raw, 4, str(tmp_path / "toy"), dtype="float32", init_scale=5.0)
        core = EngineCore(folder, "float32", page_size=4, num_pages=32, max_requests=3)
        assert len(core.cache.groups) == 1 and core.cache.slots.num_slots == 3
        rng = random.Random(2)
        reqs = {"a": [rng.randrange(300) for _ in range(21)], "b": [rng.randrange(300) for _ in range(9)]}

        # plain computation of the same model, whole sequences
        w = P.read_safetensors(os.path.join(folder, "model.safetensors"))

        def plain(ids):
            t = len(ids)
            hdn = P.embedding(ids, w["embed_tokens.weight"])
            for layer in (0, 1, 0):
                p = f"layers.{layer}."
                x = P.rms_norm(hdn, w[p + "ln1.weight"], 1e-5)
                if layer == 0:
                    s, ys = torch.zeros(48), []
                    for i in range(t):
                        s = 0.8 * s + x[i]
                        ys.append(s @ w[p + "mixer.mix.weight"].t())
                    y = torch.stack(ys)
                else:
                    q = P.linear(x, w[p + "mixer.q_proj.weight"], w[p + "mixer.q_proj.bias"]).view(t, 4, 16)
                    k = P.linear(x, w[p + "mixer.k_proj.weight"], w[p + "mixer.k_proj.bias"]).view(t, 2, 16)
                    v = P.linear(x, w[p + "mixer.v_proj.weight"], w[p + "mixer.v_proj.bias"]).view(t, 2, 16)
                    pos = torch.arange(t)
                    a = P.attention(P.rope(q, pos, 10000.0), P.rope(k, pos, 10000.0), v, 0.25)
                    y = P.linear(a.reshape(t, 64), w[p + "mixer.o_proj.weight"], None)
                hdn = hdn + y
                x = P.rms_norm(hdn, w[p + "ln2.weight"], 1e-5)
                hdn = hdn + P.linear(P.swiglu(P.linear(x, w[p + "mlp.gate_proj.weight"], None),
                                              P.linear(x, w[p + "mlp.up_proj.weight"], None)),
                                     w[p + "mlp.down_proj.weight"], None)
            return P.linear(P.rms_norm(hdn, w["norm.weight"], 1e-5), w["embed_tokens.weight"], None)

        ref = {rid: plain(ids) for rid, ids in reqs.items()}
        # portions of both requests in the same steps; the state has to carry over between steps
        cuts = [[("a", 5), ("b", 2)], [("a", 1), ("b", 6)], [("a", 9)], [("b", 1), ("a", 6)]]
        done = {"a": 0, "b": 0}
        worst = 0.0
        for cut in cuts:
            entries = [StepEntry(rid, reqs[rid][done[rid]:done[rid] + n], list(range(n))) for rid, n in cut]
            logits = core.step(entries).cpu()
            row = 0
            for rid, n in cut:
                worst = max(worst, float((logits[row:row + n] - ref[rid][done[rid]:done[rid] + n]).abs().max()))
                row += n
                done[rid] += n
        assert done == {"a": 21, "b": 9} and worst < 2e-4, worst
        core.end("a"), core.end("b")
        core.cache.check()
        assert core.cache.slots.num_free_slots == 3
    finally:
        unregister_architecture("ToyForCausalLM")
        unregister("mixer", "toy_decay")
