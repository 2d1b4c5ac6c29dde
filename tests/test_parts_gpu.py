"""Each part of a layer alone against its plain formula, and toy parts defined here (a mixer with state of its
own, a feed-forward that routes tokens to experts, another position rule), registered, built into models, loaded
and stepped without a change to the framework's files."""
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
        # the mixer loops over the step's segments on the host, so no step of this model is captured; the engine
        # says which part that is due to
        assert not core.capture_safe and core.capture_blockers == ["layers.0.mixer.DecayMixer"]
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


def test_toy_arrangement_with_two_mixers_and_no_feed_forward(tmp_path):
    """A layer is whatever parts its spec names under role names: here one with an attention mixer and a stateful toy
    mixer side by side and no feed-forward at all, put together by an arrangement that the test registers.  Each
    mixer has a cache of its own in each call of the layer (pages for one, a state slot for the other), and the
    run order names that layer twice."""
    from zedinfer_b200.cache import StateNeed
    from zedinfer_b200.config import (LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture,
                                      unregister_architecture)
    from zedinfer_b200.engine.core import EngineCore, StepEntry
    from zedinfer_b200.parts import Block, Mixer, register_block, register_mixer, unregister
    from zedinfer_b200.weights import TensorSpec, write_random_model

    @register_mixer("toy_decay2")
    class DecayMixer(Mixer):
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

    @register_block("toy_side_by_side")
    class SideBySide(Block):
        """h = h + attention(norm1(h)) + decay(norm1(h)); nothing else."""

        def forward(self, stream, ctx, caches, owns_cache):
            normed = ctx.empty(*stream.h.shape)
            self.norms["norm1"].forward_residual(stream, normed)
            a = self.mixer.forward(normed, ctx, caches["mixer"], owns_cache)
            b = self.parts()["mixer2"].forward(normed, ctx, caches["mixer2"], owns_cache)
            stream.delta = a + b

    def build_spec(raw):
        h = raw["hidden_size"]
        norm = PartSpec("rmsnorm", {"size": h, "eps": raw["eps"]})
        ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": raw["inter"]})
        attn = PartSpec("attention", {"hidden_size": h, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                      "position": PartSpec("rope", {"head_dim": 16, "theta": 10000.0})})
        toy = PartSpec("toy_decay2", {"hidden_size": h, "decay": raw["decay"]})
        both = LayerSpec("toy_side_by_side", attn, None, {"norm1": norm}, {"mixer": "attn.", "mixer2": "decay.", "norm1": "ln1."},
                         extra={"mixer2": ("mixer", toy)})
        usual = LayerSpec("pre_norm", attn, ffn, {"norm1": norm, "norm2": norm},
                          {"mixer": "mixer.", "ffn": "mlp.", "norm1": "ln1.", "norm2": "ln2."})
        return ModelSpec("Toy4ForCausalLM", raw["vocab_size"], h, (both, usual), (LayerCall(0), LayerCall(1), LayerCall(0)),
                         norm, True, raw["max_position_embeddings"])

    register_architecture("Toy4ForCausalLM", model_types=("toy4",), parse=lambda raw: raw, build_spec=build_spec)
    try:
        raw = {"architectures": ["Toy4ForCausalLM"], "hidden_size": 48, "inter": 100, "vocab_size": 300, "eps": 1e-5,
               "decay": 0.7, "max_position_embeddings": 128}
        folder = write_random_model(raw, 6, str(tmp_path / "toy4"), dtype="float32", init_scale=5.0)
        core = EngineCore(folder, "float32", page_size=4, num_pages=32, max_requests=3)
        # three calls with pages (one group of three), two of them with a state slot as well
        assert len(core.cache.groups) == 1 and len(core.cache.groups[0].calls) == 3 and core.cache.slots.num_slots == 3
        assert set(core.views) == {0, 1, 2, (0, "mixer2"), (2, "mixer2")}
        w = P.read_safetensors(os.path.join(folder, "model.safetensors"))
        assert "layers.0.decay.mix.weight" in w and "layers.0.attn.q_proj.weight" in w and "layers.0.ln2.weight" not in w

        def attention(x, p, t):
            q = P.linear(x, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).view(t, 4, 16)
            k = P.linear(x, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(t, 2, 16)
            v = P.linear(x, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(t, 2, 16)
            pos = torch.arange(t)
            a = P.attention(P.rope(q, pos, 10000.0), P.rope(k, pos, 10000.0), v, 0.25)
            return P.linear(a.reshape(t, 64), w[p + "o_proj.weight"], None)

        def plain(ids):
            t = len(ids)
            hdn = P.embedding(ids, w["embed_tokens.weight"])
            for layer in (0, 1, 0):
                p = f"layers.{layer}."
                x = P.rms_norm(hdn, w[p + "ln1.weight"], 1e-5)
                if layer == 0:
                    s, ys = torch.zeros(48), []
                    for i in range(t):
                        s = 0.7 * s + x[i]
                        ys.append(s @ w[p + "decay.mix.weight"].t())
                    hdn = hdn + (attention(x, p + "attn.", t) + torch.stack(ys))
                else:
                    hdn = hdn + attention(x, p + "mixer.", t)
                    x = P.rms_norm(hdn, w[p + "ln2.weight"], 1e-5)
                    hdn = hdn + P.linear(P.swiglu(P.linear(x, w[p + "mlp.gate_proj.weight"], None),
                                                  P.linear(x, w[p + "mlp.up_proj.weight"], None)),
                                         w[p + "mlp.down_proj.weight"], None)
            return P.linear(P.rms_norm(hdn, w["norm.weight"], 1e-5), w["embed_tokens.weight"], None)

        rng = random.Random(8)
        reqs = {"a": [rng.randrange(300) for _ in range(19)], "b": [rng.randrange(300) for _ in range(11)]}
        ref = {rid: plain(ids) for rid, ids in reqs.items()}
        cuts = [[("a", 4), ("b", 3)], [("b", 1), ("a", 7)], [("a", 1), ("b", 7)], [("a", 7)]]
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
        assert done == {"a": 19, "b": 11} and worst < 2e-4, worst
        core.end("a"), core.end("b")
        core.cache.check()
        assert core.cache.slots.num_free_slots == 3 and core.cache.groups[0].pool.num_used == 0
        # the usual arrangement says which of its parts a layer lacks
        bad = LayerSpec("pre_norm", PartSpec("toy_decay2", {"hidden_size": 48, "decay": 0.5}), None,
                        {"norm1": PartSpec("rmsnorm", {"size": 48, "eps": 1e-5})}, {})
        from zedinfer_b200.engine.model import Model
        with pytest.raises(ValueError, match="ffn.*norm2"):
            Model(ModelSpec("Toy4ForCausalLM", 300, 48, (bad,), (LayerCall(0),), PartSpec("rmsnorm", {"size": 48, "eps": 1e-5}), True, 128))
    finally:
        unregister_architecture("Toy4ForCausalLM")
        unregister("mixer", "toy_decay2")
        unregister("block", "toy_side_by_side")


# ---- a toy architecture with a routed feed-forward and another position rule ------------------------------
def test_toy_routed_feed_forward_and_toy_position_rule(tmp_path):
    """A feed-forward that routes each token to one of three experts (float32 router logits, top-1) and a position
    rule that is not the model's (rotation by half the position: "interpolated" angles), both defined here,
    registered, and used by a model of two layers whose second layer keeps the dense feed-forward and the usual
    rule.  Logits under changing portions equal a plain computation of whole sequences."""
    from zedinfer_b200 import ops
    from zedinfer_b200.config import (LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture,
                                      unregister_architecture)
    from zedinfer_b200.engine.core import EngineCore, StepEntry
    from zedinfer_b200.parts import FeedForward, PositionEncoding, register_feed_forward, register_position, unregister
    from zedinfer_b200.weights import TensorSpec, write_random_model

    @register_feed_forward("toy_top1")
    class Top1Experts(FeedForward):
        """y = expert_e(x) with e = argmax(router(x)); an expert is down(silu(up(x)))."""

        def __init__(self, hidden_size, inner, experts):
            self.h, self.inner, self.e = hidden_size, inner, experts

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec((self.e, self.h))}
            for i in range(self.e):
                specs[f"experts.{i}.up.weight"] = TensorSpec((self.inner, self.h))
                specs[f"experts.{i}.down.weight"] = TensorSpec((self.h, self.inner))
            return specs

        def bind(self, tensors):
            self.router = tensors["router.weight"].float()
            self.up = [tensors[f"experts.{i}.up.weight"] for i in range(self.e)]
            self.down = [tensors[f"experts.{i}.down.weight"] for i in range(self.e)]

        def forward(self, x, ctx):
            logits = torch.empty((x.shape[0], self.e), dtype=torch.float32, device=x.device)
            ops.linear(x.float(), self.router, None, logits)                  # router logits in float32
            choice = torch.argmax(logits, dim=1)
            out = torch.zeros_like(x)
            for i in range(self.e):
                rows = torch.nonzero(choice == i).flatten()
                if rows.numel() == 0:
                    continue
                xi = x[rows].contiguous()
                mid = torch.empty((rows.numel(), self.inner), dtype=x.dtype, device=x.device)
                ops.linear(xi, self.up[i], None, mid)
                mid = (mid.float() * torch.sigmoid(mid.float())).to(x.dtype)
                yi = torch.empty((rows.numel(), self.h), dtype=x.dtype, device=x.device)
                ops.linear(mid, self.down[i], None, yi)
                out[rows] = yi
            return out

    @register_position("toy_half_rope")
    class HalfRope(PositionEncoding):
        """Rotate-half with angle = (position / 2) * inv_freq: the framework's rotation kernel, other constants."""

        def __init__(self, head_dim, theta):
            self.head_dim, self.theta, self._inv = head_dim, theta, None

        def rotate_append(self, qkv, q_out, cache, ctx, n_heads, n_kv_heads, head_dim, write_kv):
            if self._inv is None:
                expo = torch.arange(0, head_dim, 2, dtype=torch.float32) / float(head_dim)
                self._inv = (0.5 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), expo)).to(qkv.device)
            ops.rope_append(qkv, q_out, cache.tensor, ctx.tables[cache.group], ctx.tok_seg, ctx.positions, self._inv,
                            n_heads, n_kv_heads, head_dim, cache.page_size, cache.page_stride, cache.kv_stride,
                            write_kv=write_kv)

    def build_spec(raw):
        h = raw["hidden_size"]
        norm = PartSpec("rmsnorm", {"size": h, "eps": raw["eps"]})

        def attn(position):
            return PartSpec("attention", {"hidden_size": h, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                          "position": PartSpec(position, {"head_dim": 16, "theta": 10000.0})})
        routed = PartSpec("toy_top1", {"hidden_size": h, "inner": raw["inter"], "experts": 3})
        dense = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": raw["inter"]})
        prefixes = {"mixer": "mixer.", "ffn": "mlp.", "norm1": "ln1.", "norm2": "ln2."}
        layers = (LayerSpec("pre_norm", attn("toy_half_rope"), routed, {"norm1": norm, "norm2": norm}, prefixes),
                  LayerSpec("pre_norm", attn("rope"), dense, {"norm1": norm, "norm2": norm}, prefixes))
        return ModelSpec("Toy2ForCausalLM", raw["vocab_size"], h, layers, (LayerCall(0), LayerCall(1)), norm, True,
                         raw["max_position_embeddings"])

    register_architecture("Toy2ForCausalLM", model_types=("toy2",), parse=lambda raw: raw, build_spec=build_spec)
    try:
        raw = {"architectures": ["Toy2ForCausalLM"], "hidden_size": 48, "inter": 72, "vocab_size": 211, "eps": 1e-5,
               "max_position_embeddings": 128}
        folder = write_random_model(raw, 6, str(tmp_path / "toy2"), dtype="float32", init_scale=5.0)
        core = EngineCore(folder, "float32", page_size=4, num_pages=32, max_requests=3)
        rng = random.Random(8)
        reqs = {"a": [rng.randrange(211) for _ in range(23)], "b": [rng.randrange(211) for _ in range(10)]}
        w = P.read_safetensors(os.path.join(folder, "model.safetensors"))

        def plain(ids):
            t = len(ids)
            pos = torch.arange(t)
            hdn = P.embedding(ids, w["embed_tokens.weight"])
            for layer in (0, 1):
                p = f"layers.{layer}."
                x = P.rms_norm(hdn, w[p + "ln1.weight"], 1e-5)
                q = P.linear(x, w[p + "mixer.q_proj.weight"], w[p + "mixer.q_proj.bias"]).view(t, 4, 16)
                k = P.linear(x, w[p + "mixer.k_proj.weight"], w[p + "mixer.k_proj.bias"]).view(t, 2, 16)
                v = P.linear(x, w[p + "mixer.v_proj.weight"], w[p + "mixer.v_proj.bias"]).view(t, 2, 16)
                where = pos.float() / 2.0 if layer == 0 else pos
                a = P.attention(P.rope(q, where, 10000.0), P.rope(k, where, 10000.0), v, 0.25)
                hdn = hdn + P.linear(a.reshape(t, 64), w[p + "mixer.o_proj.weight"], None)
                x = P.rms_norm(hdn, w[p + "ln2.weight"], 1e-5)
                if layer == 0:
                    choice = torch.argmax(P.linear(x, w[p + "mlp.router.weight"], None), dim=1)
                    y = torch.zeros_like(x)
                    for i in range(t):
                        e = int(choice[i])
                        mid = P.linear(x[i:i + 1], w[p + f"mlp.experts.{e}.up.weight"], None)
                        y[i] = P.linear(mid * torch.sigmoid(mid), w[p + f"mlp.experts.{e}.down.weight"], None)[0]
                else:
                    y = P.linear(P.swiglu(P.linear(x, w[p + "mlp.gate_proj.weight"], None),
                                          P.linear(x, w[p + "mlp.up_proj.weight"], None)),
                                 w[p + "mlp.down_proj.weight"], None)
                hdn = hdn + y
            return P.linear(P.rms_norm(hdn, w["norm.weight"], 1e-5), w["embed_tokens.weight"], None), None

        ref = {rid: plain(ids)[0] for rid, ids in reqs.items()}
        cuts = [[("a", 6), ("b", 3)], [("a", 2), ("b", 7)], [("a", 11)], [("a", 4)]]
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
        assert done == {"a": 23, "b": 10} and worst < 2e-4, worst
        core.end("a"), core.end("b")
        core.cache.check()
    finally:
        unregister_architecture("Toy2ForCausalLM")
        unregister("ffn", "toy_top1")
        unregister("position", "toy_half_rope")


# ---- a toy architecture whose two ends and whose positions are not the built-in ones ----------------------
def test_toy_embedding_head_and_two_position_axes(tmp_path):
    """An embedding that scales its rows, a head with a bias of its own, and a position rule that reads the second
    of two position numbers per token, all defined here and named in the ModelSpec (``embedding=``, ``head=``,
    ``position_width=2``); nothing under ``zedinfer_b200/`` knows them.  Logits under changing portions equal a plain
    computation; greedy generation through the engine with captured decode steps (positions of both axes then move
    on the device, step after step) gives the plain tokens."""
    from zedinfer_b200 import GenerationConfig, SchedulerConfig, ops
    from zedinfer_b200.config import (LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture,
                                      unregister_architecture)
    from zedinfer_b200.engine import InferenceEngine
    from zedinfer_b200.engine.core import EngineCore, StepEntry
    from zedinfer_b200.parts import (Embedding, Head, PositionEncoding, register_embedding, register_head,
                                     register_position, unregister)
    from zedinfer_b200.weights import TensorSpec, write_random_model

    @register_embedding("toy_scaled_embedding")
    class ScaledEmbedding(Embedding):
        capture_safe = True

        def __init__(self, vocab_size, hidden_size, scale):
            self.v, self.h, self.scale, self.table = vocab_size, hidden_size, scale, None

        def tensor_specs(self):
            return {"tok.weight": TensorSpec((self.v, self.h))}

        def bind(self, tensors):
            self.table = tensors["tok.weight"].contiguous()

        def forward(self, ids, out):
            ops.embedding(self.table, ids, out)
            out.mul_(self.scale)

    @register_head("toy_biased_head")
    class BiasedHead(Head):
        capture_safe = True

        def __init__(self, vocab_size, hidden_size):
            self.v, self.h = vocab_size, hidden_size

        def tensor_specs(self):
            return {"out.weight": TensorSpec((self.v, self.h)), "out.bias": TensorSpec((self.v,))}

        def bind(self, tensors, embedding=None):
            assert embedding is None                      # this embedding offers nothing to tie to
            self.w, self.b = tensors["out.weight"].contiguous(), tensors["out.bias"].contiguous()

        def forward(self, x, out):
            ops.linear(x, self.w, self.b, out)

    @register_position("toy_second_axis_rope")
    class SecondAxisRope(PositionEncoding):
        """The framework's rotation kernel fed with the second position number of every token."""
        capture_safe = True

        def __init__(self, head_dim, theta):
            self.head_dim, self.theta, self._inv = head_dim, theta, None

        def rotate_append(self, qkv, q_out, cache, ctx, n_heads, n_kv_heads, head_dim, write_kv):
            assert ctx.position_axes.shape == (2, ctx.n_tokens)
            if self._inv is None:
                expo = torch.arange(0, head_dim, 2, dtype=torch.float32) / float(head_dim)
                self._inv = (1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), expo)).to(qkv.device)
            ops.rope_append(qkv, q_out, cache.tensor, ctx.tables[cache.group], ctx.tok_seg, ctx.position_axes[1],
                            self._inv, n_heads, n_kv_heads, head_dim, cache.page_size, cache.page_stride,
                            cache.kv_stride, write_kv=write_kv)

    H, V, INTER, SCALE = 48, 157, 80, 3.0

    def build_spec(raw):
        norm = PartSpec("rmsnorm", {"size": H, "eps": 1e-5})
        attn = PartSpec("attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                      "position": PartSpec("toy_second_axis_rope", {"head_dim": 16, "theta": 500.0})})
        dense = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": INTER})
        prefixes = {"mixer": "mixer.", "ffn": "mlp.", "norm1": "ln1.", "norm2": "ln2."}
        layer = LayerSpec("pre_norm", attn, dense, {"norm1": norm, "norm2": norm}, prefixes)
        return ModelSpec("Toy3ForCausalLM", V, H, (layer, layer), (LayerCall(0), LayerCall(1)), norm, False,
                         raw["max_position_embeddings"],
                         embedding=PartSpec("toy_scaled_embedding", {"vocab_size": V, "hidden_size": H, "scale": SCALE}),
                         head=PartSpec("toy_biased_head", {"vocab_size": V, "hidden_size": H}), position_width=2)

    register_architecture("Toy3ForCausalLM", model_types=("toy3",), parse=lambda raw: raw, build_spec=build_spec)
    try:
        raw = {"architectures": ["Toy3ForCausalLM"], "max_position_embeddings": 128}
        folder = write_random_model(raw, 4, str(tmp_path / "toy3"), dtype="float32", init_scale=5.0)
        w = P.read_safetensors(os.path.join(folder, "model.safetensors"))
        assert "tok.weight" in w and "out.bias" in w and "embed_tokens.weight" not in w

        def plain(ids):
            t = len(ids)
            pos = torch.arange(t)
            hdn = P.embedding(ids, w["tok.weight"]) * SCALE
            for layer in (0, 1):
                p = f"layers.{layer}."
                x = P.rms_norm(hdn, w[p + "ln1.weight"], 1e-5)
                q = P.linear(x, w[p + "mixer.q_proj.weight"], w[p + "mixer.q_proj.bias"]).view(t, 4, 16)
                k = P.linear(x, w[p + "mixer.k_proj.weight"], w[p + "mixer.k_proj.bias"]).view(t, 2, 16)
                v = P.linear(x, w[p + "mixer.v_proj.weight"], w[p + "mixer.v_proj.bias"]).view(t, 2, 16)
                a = P.attention(P.rope(q, pos, 500.0), P.rope(k, pos, 500.0), v, 0.25)
                hdn = hdn + P.linear(a.reshape(t, 64), w[p + "mixer.o_proj.weight"], None)
                x = P.rms_norm(hdn, w[p + "ln2.weight"], 1e-5)
                hdn = hdn + P.linear(P.swiglu(P.linear(x, w[p + "mlp.gate_proj.weight"], None),
                                              P.linear(x, w[p + "mlp.up_proj.weight"], None)),
                                     w[p + "mlp.down_proj.weight"], None)
            return P.linear(P.rms_norm(hdn, w["norm.weight"], 1e-5), w["out.weight"], w["out.bias"])

        core = EngineCore(folder, "float32", page_size=4, num_pages=32, max_requests=3)
        assert core.capture_blockers == [] and core.spec.position_width == 2
        rng = random.Random(3)
        reqs = {"a": [rng.randrange(V) for _ in range(23)], "b": [rng.randrange(V) for _ in range(10)]}
        ref = {rid: plain(ids) for rid, ids in reqs.items()}
        done, worst = {"a": 0, "b": 0}, 0.0
        for cut in [[("a", 6), ("b", 3)], [("a", 2), ("b", 7)], [("a", 11)], [("a", 4)]]:
            entries = [StepEntry(rid, reqs[rid][done[rid]:done[rid] + n], list(range(n))) for rid, n in cut]
            logits = core.step(entries).cpu()
            row = 0
            for rid, n in cut:
                worst = max(worst, float((logits[row:row + n] - ref[rid][done[rid]:done[rid] + n]).abs().max()))
                row += n
                done[rid] += n
        assert worst < 2e-4, worst
        del core
        # greedy generation, decode steps captured, tokens handed on and both position axes moved on the device
        prompt, n_new = reqs["b"], 14
        seq, expected = list(prompt), []
        for _ in range(n_new):
            expected.append(P.greedy(plain(seq)[-1]))
            seq.append(expected[-1])
        engine = InferenceEngine.create(folder, SchedulerConfig(num_kv_pages=32, kv_block_size=4, max_batch_requests=2,
                                                                cuda_graphs=True), dtype="float32")
        out = engine.generate_tokens(prompt, GenerationConfig(max_new_tokens=n_new, ignore_eos=True))
        assert out.output_ids == expected
        graphs = list(engine.core._decode_graphs.values())
        assert graphs and all(g.ctx.position_axes.shape[0] == 2 for g in graphs)
        for g in graphs:
            axes = g.ctx.position_axes.cpu()
            assert torch.equal(axes[0], axes[1])
    finally:
        unregister_architecture("Toy3ForCausalLM")
        unregister("embedding", "toy_scaled_embedding")
        unregister("head", "toy_biased_head")
        unregister("position", "toy_second_axis_rope")
