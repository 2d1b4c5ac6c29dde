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
prompt in one forward) and ``logits_chunk5.npy`` (the prompt in portions of 5 with a growing past length).
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


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    from zedinfer_b200.weights import SafetensorsFile, canonical_name, write_random_model
    model_dir = os.path.join(HERE, "model")
    write_random_model(CONFIG, SEED, model_dir, dtype="float32", init_scale=8.0)
    g = torch.Generator().manual_seed(123)
    ids = torch.randint(0, CONFIG["vocab_size"], (TOKENS,), generator=g).tolist()
    with open(os.path.join(HERE, "ids.json"), "w") as f:
        json.dump(ids, f)
    with tempfile.TemporaryDirectory() as tmp:
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
