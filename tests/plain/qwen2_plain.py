"""A plain, slow implementation of the Qwen2 forward pass: whole sequences, no cache, one
function per part, float32 on the CPU.  It shares no code with ``zedinfer_b200``: it reads
``config.json`` with ``json`` and ``model.safetensors`` with its own few lines, and every
function is written from the formulas of the reference, cited as file:line of
tianyuxbear/zedinfer.

``tests/golden/`` holds logits that the reference's own CPU forward produced for a tiny
random model; ``tests/test_plain.py`` checks this file against them.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------
# files
# ---------------------------------------------------------------------------------------------
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """name -> float32 tensor.  8-byte header length, JSON header, raw data
    (src/frontend/loader/safetensor.cpp:105-150)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        if info["dtype"] == "F32":
            t = torch.frombuffer(bytearray(raw), dtype=torch.float32)
        elif info["dtype"] == "BF16":
            t = torch.frombuffer(bytearray(raw), dtype=torch.bfloat16).float()
        elif info["dtype"] == "F16":
            t = torch.frombuffer(bytearray(raw), dtype=torch.float16).float()
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        # strip "model." as the reference does (src/frontend/models/base.cpp:1389-1392)
        key = name[6:] if name.startswith("model.") else name
        out[key] = t.reshape(info["shape"]).clone()
    return out


def read_config(model_dir: str) -> dict:
    """Keys and defaults of src/frontend/models/base.cpp:683-720 and :807-813."""
    with open(os.path.join(model_dir, "config.json")) as f:
        j = json.load(f)
    nh = j["num_attention_heads"]
    cfg = {
        "hidden_size": j["hidden_size"],
        "intermediate_size": j["intermediate_size"],
        "vocab_size": j["vocab_size"],
        "num_hidden_layers": j["num_hidden_layers"],
        "num_attention_heads": nh,
        "num_key_value_heads": j.get("num_key_value_heads", nh),
        "head_dim": j.get("head_dim") or j["hidden_size"] // nh,
        "rms_norm_eps": j.get("rms_norm_eps", 1e-6),
        "rope_theta": j.get("rope_theta", 10000.0),
        "tie_word_embeddings": j.get("tie_word_embeddings", False),
        "use_sliding_window": j.get("use_sliding_window", False),
        "sliding_window": j.get("sliding_window", 4096),
        "max_window_layers": j.get("max_window_layers", 21),
    }
    return cfg


# ---------------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------------
def round_to(x: torch.Tensor, dtype: Optional[torch.dtype]) -> torch.Tensor:
    """Round to the storage type of activations and come back to float32 (None: keep float32)."""
    return x if dtype is None else x.to(dtype).float()


def embedding(ids: List[int], table: torch.Tensor) -> torch.Tensor:
    """hidden[n, :] = table[ids[n], :]  (src/backend/ops/embedding/cpu/embedding_cpu.cpp:19-22)"""
    return table[torch.tensor(ids, dtype=torch.long)].clone()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """rstd = 1/sqrt(sum(x^2)/H + eps); y = (w * x) * rstd
    (src/backend/ops/rms_norm/cpu/rms_norm_cpu.cpp:24-28)"""
    h = x.shape[-1]
    ss = (x * x).sum(dim=-1, keepdim=True)
    rstd = 1.0 / torch.sqrt(ss / float(h) + eps)
    return (w * x) * rstd


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """C[M,N] = A[M,K] . W[N,K]^T + bias[N]  (src/backend/ops/linear/cpu/linear_cpu.cpp:28-37)"""
    y = x @ w.t()
    return y + b if b is not None else y


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [T, heads, hd]; inv[k] = 1/theta^(2k/hd); ang = float(p)*inv[k];
    y[k] = a*cos - b*sin; y[k+half] = b*cos + a*sin, a = x[k], b = x[k+half]
    (src/backend/ops/rope/cpu/rope_cpu.cpp:32-52, :60-65)"""
    hd = x.shape[-1]
    half = hd // 2
    expo = torch.arange(0, hd, 2, dtype=torch.float32) / float(hd)
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), expo)
    ang = positions.to(torch.float32)[:, None] * inv[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
              window: Optional[int] = None) -> torch.Tensor:
    """q [T, nh, hd], k/v [T, nkv, hd] of one whole sequence starting at position 0.
    For query i and head h (kvh = h // (nh/nkv)): s_j = (q_i . k_j) * scale for j <= i
    (and j > i - window when a window is set); softmax; out = sum_j p_j v_j
    (src/backend/ops/self_attention/cpu/paged_attention_cpu.cpp:113-159)"""
    t, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    out = torch.zeros_like(q)
    for h in range(nh):
        kvh = h // group
        scores = (q[:, h, :] @ k[:, kvh, :].t()) * scale                 # [T, T]
        i = torch.arange(t)[:, None]
        j = torch.arange(t)[None, :]
        mask = j <= i
        if window is not None:
            mask &= j > i - window
        scores = scores.masked_fill(~mask, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        out[:, h, :] = (e @ v[:, kvh, :]) * (1.0 / e.sum(dim=-1, keepdim=True))
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """a = up * gate / (1 + exp(-gate))  (src/backend/ops/swiglu/cpu/swiglu_cpu.cpp:13-20)"""
    return up * gate / (1.0 + torch.exp(-gate))


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def layer_window(cfg: dict, layer: int) -> Optional[int]:
    if cfg["use_sliding_window"] and layer >= cfg["max_window_layers"]:
        return cfg["sliding_window"]
    return None


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int],
            act_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Logits [T, V] of one whole sequence (src/frontend/models/transformer_forward.cpp:58-156).

    ``act_dtype=torch.bfloat16`` rounds the outputs of projections, norms, rotation, attention
    and the activation to bfloat16 as a bfloat16 engine stores them; the residual stream and
    the logits stay float32.
    """
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps, theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    t = len(ids)
    pos = torch.arange(t)
    scale = 1.0 / math.sqrt(float(hd))                                     # transformer_forward.cpp:31
    r = lambda x: round_to(x, act_dtype)                                   # noqa: E731
    hidden = embedding(ids, w["embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        p = f"layers.{layer}."
        x = r(rms_norm(hidden, w[p + "input_layernorm.weight"], eps))
        q = r(linear(x, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.q_proj.bias"])).view(t, nh, hd)
        k = r(linear(x, w[p + "self_attn.k_proj.weight"], w[p + "self_attn.k_proj.bias"])).view(t, nkv, hd)
        v = r(linear(x, w[p + "self_attn.v_proj.weight"], w[p + "self_attn.v_proj.bias"])).view(t, nkv, hd)
        q, k = r(rope(q, pos, theta)), r(rope(k, pos, theta))
        a = r(attention(q, k, v, scale, layer_window(cfg, layer))).reshape(t, nh * hd)
        o = r(linear(a, w[p + "self_attn.o_proj.weight"], None))
        hidden = hidden + o
        x = r(rms_norm(hidden, w[p + "post_attention_layernorm.weight"], eps))
        g = r(linear(x, w[p + "mlp.gate_proj.weight"], None))
        u = r(linear(x, w[p + "mlp.up_proj.weight"], None))
        d = r(linear(r(swiglu(g, u)), w[p + "mlp.down_proj.weight"], None))
        hidden = hidden + d
    x = r(rms_norm(hidden, w["norm.weight"], eps))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["embed_tokens.weight"]   # base.cpp:411-416
    return linear(x, head, None)


def load(model_dir: str):
    return read_config(model_dir), read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---------------------------------------------------------------------------------------------
# random weights without a folder
# ---------------------------------------------------------------------------------------------
_U64 = (1 << 64) - 1


def _as_i64(v: int) -> int:
    v &= _U64
    return v - (1 << 64) if v >= (1 << 63) else v


def _splitmix(z: int) -> int:
    z &= _U64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _U64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _U64
    return z ^ (z >> 31)


def random_values(seed: int, name: str, shape, std: float, plus_one: bool = False, device="cpu") -> torch.Tensor:
    """The engine's random-weights rule, restated (the reference has none; it draws token ids only,
    src/zedinfer/profiler.cpp:79-84).  Element i of tensor ``name`` is twelve 16-bit fields of three
    splitmix64 words of (key + (3 i + j) * golden), summed and centred: ``x = (2 s - 12 * 65535) / 2^17``;
    the value is ``x * std`` (``1 + x * std`` for norm weights), float32.  Integer arithmetic up to one exact
    conversion, so ``device`` (where the arithmetic runs; the result comes back to the CPU) changes no bit."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _U64
    key = _splitmix(h ^ _splitmix(seed))
    n = 1
    for d in shape:
        n *= int(d)
    out = torch.empty(n, dtype=torch.float32, device=device)
    srl = lambda z, k: (z >> k) & ((1 << (64 - k)) - 1)                      # noqa: E731  (logical shift)
    step = 1 << 18 if str(device) == "cpu" else 1 << 24
    for lo in range(0, n, step):
        i3 = torch.arange(lo, min(lo + step, n), dtype=torch.int64, device=device) * 3
        total = torch.zeros_like(i3)
        for j in range(3):
            z = (i3 + j) * _as_i64(0x9E3779B97F4A7C15) + _as_i64(key)
            z = (z ^ srl(z, 30)) * _as_i64(0xBF58476D1CE4E5B9)
            z = (z ^ srl(z, 27)) * _as_i64(0x94D049BB133111EB)
            z = z ^ srl(z, 31)
            pairs = (z & 0x0000FFFF0000FFFF) + (srl(z, 16) & 0x0000FFFF0000FFFF)   # fields 0+1 and 2+3, side by side
            total += (pairs & 0xFFFFFFFF) + srl(pairs, 32)
        out[lo: lo + i3.numel()] = (2 * total - 12 * 65535).float() / 131072.0
    out *= float(torch.tensor(std, dtype=torch.float32))
    if plus_one:
        out += 1.0
    return out.view(tuple(shape)).cpu()


def random_weights(cfg: dict, seed: int, init_scale: float = 1.0, dtype: Optional[torch.dtype] = None,
                   device="cpu") -> Dict[str, torch.Tensor]:
    """Every tensor of a Qwen2 model of ``cfg`` (the dict of :func:`read_config`) drawn with ``seed``:
    projections, biases and embeddings N(0, 0.02 * init_scale), norm weights 1 + N(0, 0.01); ``dtype``
    rounds them as a stored model would (None: float32).  Returned as float32."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd, kd = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    shapes = {"embed_tokens.weight": (v, h), "norm.weight": (h,)}
    if not cfg["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (v, h)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"layers.{layer}."
        shapes.update({p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
                       p + "self_attn.q_proj.weight": (qd, h), p + "self_attn.q_proj.bias": (qd,),
                       p + "self_attn.k_proj.weight": (kd, h), p + "self_attn.k_proj.bias": (kd,),
                       p + "self_attn.v_proj.weight": (kd, h), p + "self_attn.v_proj.bias": (kd,),
                       p + "self_attn.o_proj.weight": (h, qd), p + "mlp.gate_proj.weight": (i, h),
                       p + "mlp.up_proj.weight": (i, h), p + "mlp.down_proj.weight": (h, i)})
    out = {}
    for name, shape in shapes.items():
        norm = name.endswith("norm.weight") or name.endswith("layernorm.weight")
        t = random_values(seed, name, shape, 0.01 if norm else 0.02 * init_scale, plus_one=norm, device=device)
        out[name] = round_to(t, dtype)
    return out


def config_from_dict(j: dict) -> dict:
    """:func:`read_config` for a config.json that is already a dict."""
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        with open(os.path.join(tmp, "config.json"), "w") as f:
            json.dump(j, f)
        return read_config(tmp)


# ---------------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------------
def greedy(logits_row: torch.Tensor) -> int:
    """Largest logit, lowest index on ties (src/backend/ops/argmax/cpu/argmax_cpu.cpp:15-19)."""
    m = logits_row.max()
    return int(torch.nonzero(logits_row == m)[0, 0])


def sampling_distribution(logits_row: torch.Tensor, temperature: float, top_k: int, top_p: float,
                          recent: Optional[List[int]] = None, repetition_penalty: float = 1.0) -> torch.Tensor:
    """Probabilities over the vocabulary after penalty, temperature, softmax, top-k, top-p and
    renormalisation (src/frontend/sampler/sampler.cpp:195-247, :410-490)."""
    z = logits_row.clone().float()
    if repetition_penalty != 1.0 and recent:
        for tid in recent:
            if 0 <= tid < z.numel():
                z[tid] = z[tid] / repetition_penalty if z[tid] > 0 else z[tid] * repetition_penalty
    z = z / temperature
    p = torch.exp(z - z.max())
    p = p / p.sum()
    order = torch.argsort(p, descending=True, stable=True)
    keep = torch.ones_like(p, dtype=torch.bool)
    if 0 < top_k < p.numel():
        kth = p[order[top_k - 1]]
        keep &= p >= kth
    if top_p < 1.0:
        sp = p[order] * keep[order]
        cum = torch.cumsum(sp, 0)
        cutoff = int(torch.nonzero(cum >= top_p)[0, 0]) + 1 if bool((cum >= top_p).any()) else p.numel()
        thr = p[order[cutoff - 1]]
        keep &= p >= thr
    out = torch.where(keep, p, torch.zeros_like(p))
    return out / out.sum()


def pick_from(dist: torch.Tensor, u: float) -> int:
    """First index, in index order, whose running sum exceeds u."""
    cum = torch.cumsum(dist.double(), 0)
    idx = torch.nonzero(cum > u * float(cum[-1]))
    return int(idx[0, 0]) if idx.numel() else int(torch.nonzero(dist > 0)[-1, 0])
