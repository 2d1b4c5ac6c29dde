#!/usr/bin/env python3
"""Makes the files of this folder: logits of tianyuxbear/zedinfer's own CPU forward for a tiny random
Qwen2 model.

The reference's transformer_forward, PagedForwardContext, BlockPool, tensor/core/device layers and its
CPU kernels (src/frontend/models/transformer_forward.cpp, src/frontend/models/paged_forward_context.cpp,
src/backend/kvcache/block_pool.cpp, src/backend/ops/*/cpu/*.cpp, ...) are compiled unmodified with g++;
``ref_harness/`` holds what its build system would provide: a no-op stand-in for the plog logging
headers (its third_party submodules are empty), two stub symbols for GPU/MoE-only functions that this
path never calls, and a ``main.cpp`` that feeds weights and token ids in and writes logits out.

    python tests/golden/make_golden.py /path/to/zedinfer

writes ``model/`` (config.json, model.safetensors, float32), ``ids.json``, ``logits_whole.npy`` (the whole
prompt in one forward), ``logits_chunk5.npy`` (the prompt in portions of 5 with a growing past length) and
``sampler_cases.json`` (rows of logits with sampling options, and what the reference's own sampler keeps of them:
tokens and renormalised probabilities after repetition penalty, temperature, softmax, top-k and top-p).
tests/test_plain.py compares the plain implementation with them.
"""
import glob
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 2, "hidden_size": 32,
    "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 48, "vocab_size": 64,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 128,
}
SEED, TOKENS, BLOCK = 0, 24, 4


def build(ref: str, out_dir: str) -> str:
    nj = None
    for cand in glob.glob(os.path.join(sys.prefix, "lib", "python*", "site-packages", "include", "cudnn_frontend",
                                       "thirdparty")):
        if os.path.isfile(os.path.join(cand, "nlohmann", "json.hpp")):
            nj = cand
    if nj is None:
        raise SystemExit("nlohmann/json.hpp not found (the reference's nlohmann_json submodule is empty)")
    src = [f"{ref}/src/frontend/models/{n}.cpp" for n in ("transformer_forward", "paged_forward_context", "qwen2")]
    src += [f"{ref}/src/zedinfer/batch_context.cpp", f"{ref}/src/backend/kvcache/block_pool.cpp",
            f"{ref}/src/backend/tensor/tensor.cpp", f"{ref}/src/backend/device/runtime_api.cpp",
            f"{ref}/src/backend/device/cpu/cpu_runtime_api.cpp", f"{ref}/src/backend/ops/rearrange/op.cpp",
            f"{ref}/src/utils/types.cpp"]
    src += glob.glob(f"{ref}/src/backend/core/*/*.cpp") + glob.glob(f"{ref}/src/backend/ops/rearrange/cpu/*.cpp")
    for op in ("add", "embedding", "linear", "rms_norm", "rope", "swiglu", "self_attention", "argmax"):
        src.append(f"{ref}/src/backend/ops/{op}/op.cpp")
        src += [f for f in glob.glob(f"{ref}/src/backend/ops/{op}/cpu/*.cpp") if "onednn" not in f]
    harness = os.path.join(HERE, "ref_harness")
    exe = os.path.join(out_dir, "ref_forward")
    cmd = ["g++", "-std=c++17", "-O2", "-march=native", "-fopenmp", "-Wno-unknown-pragmas",
           "-I", os.path.join(harness, "shim"), "-I", f"{ref}/include", "-I", nj,
           os.path.join(harness, "main.cpp"), os.path.join(harness, "stubs.cpp")] + sorted(src) + ["-o", exe]
    subprocess.run(cmd, check=True)
    return exe


SAMPLER_VOCAB = 97
SAMPLER_CASES = [      # temperature, top_k, top_p, repetition_penalty, recently generated tokens
    (0.7, 0, 1.0, 1.0, []), (1.0, 5, 1.0, 1.0, []), (0.8, 0, 0.9, 1.0, []), (1.3, 20, 0.6, 1.0, []),
    (1.0, 0, 1.0, 1.3, [3, 50, 96]), (0.6, 12, 0.85, 1.5, [7, 7, 21, 60, 0]), (2.0, 1, 1.0, 1.0, []),
    (0.9, 96, 0.999, 1.1, [1, 2, 3, 4, 5, 6, 7, 8]),
]


def make_sampler_golden(ref: str, nj: str, tmp: str) -> None:
    """The reference's own GeneralSampler::truncatedDist (src/frontend/sampler/sampler.cpp:195-247), compiled
    unmodified for the CPU, on a few rows of logits: writes ``sampler_cases.json`` (inputs and its answers)."""
    src = [f"{ref}/src/frontend/sampler/sampler.cpp", f"{ref}/src/backend/tensor/tensor.cpp",
           f"{ref}/src/backend/device/runtime_api.cpp", f"{ref}/src/backend/device/cpu/cpu_runtime_api.cpp",
           f"{ref}/src/backend/ops/rearrange/op.cpp", f"{ref}/src/utils/types.cpp", f"{ref}/src/backend/ops/sample/op.cpp",
           f"{ref}/src/backend/ops/argmax/op.cpp"]
    src += glob.glob(f"{ref}/src/backend/core/*/*.cpp") + glob.glob(f"{ref}/src/backend/ops/rearrange/cpu/*.cpp")
    src += glob.glob(f"{ref}/src/backend/ops/argmax/cpu/*.cpp")
    harness = os.path.join(HERE, "ref_harness")
    exe = os.path.join(tmp, "ref_sampler")
    subprocess.run(["g++", "-std=c++17", "-O2", "-march=native", "-fopenmp", "-Wno-unknown-pragmas",
                    "-I", os.path.join(harness, "shim"), "-I", f"{ref}/include", "-I", nj,
                    os.path.join(harness, "sampler_main.cpp")] + sorted(src) + ["-o", exe], check=True)
    g = torch.Generator().manual_seed(321)
    cases = []
    lines = [f"vocab {SAMPLER_VOCAB}"]
    for temperature, top_k, top_p, penalty, recent in SAMPLER_CASES:
        logits = (torch.randn(SAMPLER_VOCAB, generator=g) * 2.5).tolist()
        lines.append(f"case {temperature} {top_k} {top_p} {penalty} {len(recent)} " + " ".join(map(str, recent)))
        lines.append(" ".join(repr(float(np.float32(v))) for v in logits))
        cases.append({"temperature": temperature, "top_k": top_k, "top_p": top_p, "repetition_penalty": penalty,
                      "recent": recent, "logits": [float(np.float32(v)) for v in logits]})
    with open(os.path.join(tmp, "cases.txt"), "w") as f:
        f.write("\n".join(lines) + "\n")
    subprocess.run([exe, os.path.join(tmp, "cases.txt"), os.path.join(tmp, "dist.txt")], check=True)
    with open(os.path.join(tmp, "dist.txt")) as f:
        rows = f.read().split("\n")
    i = 0
    for case in cases:
        _, _, n = rows[i].split()
        kept = [rows[i + 1 + k].split() for k in range(int(n))]
        case["kept_tokens"] = [int(t) for t, _ in kept]
        case["kept_probs"] = [float(p) for _, p in kept]
        i += 1 + int(n)
    with open(os.path.join(HERE, "sampler_cases.json"), "w") as f:
        json.dump({"vocab": SAMPLER_VOCAB, "cases": cases}, f)
    print("sampler_cases", [len(c["kept_tokens"]) for c in cases])


def find_nlohmann() -> str:
    for cand in glob.glob(os.path.join(sys.prefix, "lib", "python*", "site-packages", "include", "cudnn_frontend",
                                       "thirdparty")):
        if os.path.isfile(os.path.join(cand, "nlohmann", "json.hpp")):
            return cand
    raise SystemExit("nlohmann/json.hpp not found (the reference's nlohmann_json submodule is empty)")


def main():
    if len(sys.argv) != 2 or not os.path.isdir(sys.argv[1]):
        sys.exit("usage: make_golden.py <checkout of tianyuxbear/zedinfer>")
    ref = sys.argv[1]
    from zedinfer_b200.weights import SafetensorsFile, canonical_name, write_random_model
    model_dir = os.path.join(HERE, "model")
    write_random_model(CONFIG, SEED, model_dir, dtype="float32", init_scale=8.0)
    g = torch.Generator().manual_seed(123)
    ids = torch.randint(0, CONFIG["vocab_size"], (TOKENS,), generator=g).tolist()
    with open(os.path.join(HERE, "ids.json"), "w") as f:
        json.dump(ids, f)
    with tempfile.TemporaryDirectory() as tmp:
        make_sampler_golden(ref, find_nlohmann(), tmp)
        exe = build(ref, tmp)
        st = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
        c = CONFIG
        lines = [f"config {c['hidden_size']} {c['intermediate_size']} {c['vocab_size']} {c['num_hidden_layers']} "
                 f"{c['num_attention_heads']} {c['num_key_value_heads']} {c['head_dim']} {c['rms_norm_eps']} "
                 f"{c['rope_theta']} {int(c['tie_word_embeddings'])}", "ids " + " ".join(map(str, ids))]
        with open(os.path.join(tmp, "weights.bin"), "wb") as wb:
            for raw, e in st.entries.items():
                t = e.load().float().contiguous()
                lines.append(f"tensor {canonical_name(raw)} {t.dim()} " + " ".join(map(str, t.shape)))
                wb.write(t.numpy().tobytes())
        with open(os.path.join(tmp, "index.txt"), "w") as f:
            f.write("\n".join(lines) + "\n")
        for name, extra in (("logits_whole", []), ("logits_chunk5", ["5"])):
            out = os.path.join(tmp, name + ".bin")
            subprocess.run([exe, os.path.join(tmp, "index.txt"), os.path.join(tmp, "weights.bin"), out, str(BLOCK)] + extra,
                           check=True)
            arr = np.fromfile(out, dtype="<f4").reshape(TOKENS, CONFIG["vocab_size"])
            np.save(os.path.join(HERE, name + ".npy"), arr)
            print(name, arr.shape, float(np.abs(arr).max()))


if __name__ == "__main__":
    main()
