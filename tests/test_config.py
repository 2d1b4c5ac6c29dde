"""Configuration: config.json keys, defaults, errors, the registry, and the spec it builds."""
import json
import os

import pytest

import tiny
from zedinfer_b200.config import (ConfigError, GenerationConfig, LayerCall, ModelSpec, SchedulerConfig,
                                  load_model_config, register_architecture, resolve_architecture,
                                  resolve_max_new_tokens, supported_architectures, unregister_architecture)
from zedinfer_b200.models.qwen2 import build_qwen2_spec, parse_qwen2_config


def test_defaults_follow_the_reference():
    raw = {"architectures": ["Qwen2ForCausalLM"], "hidden_size": 64, "intermediate_size": 100, "vocab_size": 50,
           "num_hidden_layers": 2, "num_attention_heads": 4, "max_position_embeddings": 128}
    c = parse_qwen2_config(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.tie_word_embeddings is False and c.torch_dtype == "bfloat16"
    assert c.eos_token_ids == (151643,) and c.bos_token_id == 151643
    assert c.use_sliding_window is False and c.sliding_window == 4096 and c.max_window_layers == 21


def test_eos_as_list_and_head_dim_given():
    raw = dict(tiny.TINY_D, eos_token_id=[5, 9])
    c = parse_qwen2_config(raw)
    assert c.eos_token_ids == (5, 9)
    assert c.head_dim == 128 and c.q_dim == 12 * 128 and c.kv_dim == 256


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "vocab_size", "num_hidden_layers",
                                 "num_attention_heads", "max_position_embeddings"])
def test_missing_required_key_is_named(key):
    raw = dict(tiny.TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        parse_qwen2_config(raw)


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"rope_theta": -1.0}, "rope_theta"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"torch_dtype": "int8"}, "torch_dtype"),
    ({"eos_token_id": "x"}, "eos_token_id"),
    ({"use_sliding_window": True, "sliding_window": 0}, "sliding_window"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
])
def test_bad_values_are_refused(patch, word):
    raw = dict(tiny.TINY_A)
    raw.update(patch)
    with pytest.raises(ConfigError, match=word):
        parse_qwen2_config(raw)


def test_registry_by_architecture_and_by_model_type():
    assert "Qwen2ForCausalLM" in supported_architectures()
    assert resolve_architecture({"architectures": ["Qwen2ForCausalLM"]}).name == "Qwen2ForCausalLM"
    assert resolve_architecture({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})


def test_spec_layer_by_layer():
    spec = build_qwen2_spec(parse_qwen2_config(tiny.TINY_C))
    assert len(spec.layers) == 3 and [c.layer for c in spec.schedule] == [0, 1, 2]
    windows = [l.mixer.params["window"] for l in spec.layers]
    assert windows == [None, 24, 24]
    m = spec.layers[0].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (6, 3, 48)
    assert m["qkv_bias"] is True and m["out_bias"] is False
    assert m["position"].params == {"head_dim": 48, "theta": 50000.0}
    assert spec.layers[0].norms["norm1"].params["eps"] == 1e-4
    assert spec.layers[0].ffn.params["intermediate_size"] == 200
    assert not spec.tie_word_embeddings
    assert build_qwen2_spec(parse_qwen2_config(tiny.TINY_A)).tie_word_embeddings


def test_schedule_validation():
    spec = build_qwen2_spec(parse_qwen2_config(tiny.TINY_A))
    import dataclasses
    ok = dataclasses.replace(spec, schedule=(LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache_of=1)))
    ok.validate()
    with pytest.raises(ValueError, match="layer 5"):
        dataclasses.replace(spec, schedule=(LayerCall(5),)).validate()
    with pytest.raises(ValueError, match="earlier"):
        dataclasses.replace(spec, schedule=(LayerCall(0, cache_of=0),)).validate()
    with pytest.raises(ValueError, match="borrows"):
        dataclasses.replace(spec, schedule=(LayerCall(0), LayerCall(1, cache_of=0), LayerCall(0, cache_of=1))).validate()


def test_load_model_config_errors(tmp_path):
    with pytest.raises(ConfigError, match="Failed to open config file"):
        load_model_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_model_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_B))
    arch, cfg, spec = load_model_config(str(tmp_path))
    assert arch.name == "Qwen2ForCausalLM" and cfg.vocab_size == 1000 and spec.vocab_size == 1000


def test_another_architecture_can_be_registered():
    def parse(raw):
        return parse_qwen2_config(dict(raw, model_type="qwen2"))
    register_architecture("ToyForCausalLM", model_types=("toy",), parse=parse, build_spec=build_qwen2_spec)
    try:
        assert resolve_architecture({"model_type": "toy"}).name == "ToyForCausalLM"
    finally:
        unregister_architecture("ToyForCausalLM")
    with pytest.raises(ConfigError):
        resolve_architecture({"model_type": "toy"})


def test_engine_options():
    SchedulerConfig().validate()
    assert SchedulerConfig().max_batch_tokens == 2048 and SchedulerConfig().max_prefill_tokens == 2048
    assert SchedulerConfig().max_batch_requests == 64 and SchedulerConfig().kv_block_size == 16
    with pytest.raises(ValueError):
        SchedulerConfig(on_exhaust="swap").validate()
    with pytest.raises(ValueError):
        GenerationConfig(use_argmax=False, temperature=0.0).validate()
    with pytest.raises(ValueError):
        GenerationConfig(use_argmax=False, top_p=0.0).validate()
    with pytest.raises(ValueError):
        GenerationConfig(max_new_tokens=-1).validate()
    assert resolve_max_new_tokens(0, 10, 100) == 90
    assert resolve_max_new_tokens(500, 10, 100) == 90
    assert resolve_max_new_tokens(5, 10, 100) == 5
    with pytest.raises(ValueError, match="no room"):
        resolve_max_new_tokens(5, 100, 100)


# ---- the engine's default sampling (src/zedinfer/engine.cpp:49-126) ---------------------------------------
def _gen_folder(tmp_path, body):
    import json
    (tmp_path / "generation_config.json").write_text(body if isinstance(body, str) else json.dumps(body))
    return str(tmp_path)


def test_sampling_defaults_follow_generation_config_json(tmp_path):
    from zedinfer_b200.config import sampling_defaults
    assert sampling_defaults(None, {}).use_argmax                         # no folder
    assert sampling_defaults(str(tmp_path), {}).use_argmax                # no file
    d = _gen_folder(tmp_path, {"do_sample": True, "temperature": 0.6, "top_k": 20, "top_p": 0.95})
    g = sampling_defaults(d, {})
    assert (g.use_argmax, g.temperature, g.top_k, g.top_p, g.repetition_penalty, g.seed) == (False, 0.6, 20, 0.95, 1.0, 0)
    assert g.has_sampling_override
    g = sampling_defaults(_gen_folder(tmp_path, {"do_sample": True, "repetition_penalty": 1.1, "seed": 7}), {})
    assert (g.use_argmax, g.temperature, g.repetition_penalty, g.seed) == (False, 1.0, 1.1, 7)
    assert sampling_defaults(_gen_folder(tmp_path, {"do_sample": False, "temperature": 0.6}), {}).use_argmax
    assert sampling_defaults(_gen_folder(tmp_path, {"temperature": 0.6}), {}).use_argmax       # do_sample absent
    assert sampling_defaults(_gen_folder(tmp_path, "{ not json"), {}).use_argmax
    assert sampling_defaults(_gen_folder(tmp_path, {"do_sample": True, "top_p": 1.5}), {}).use_argmax   # does not validate
    assert sampling_defaults(_gen_folder(tmp_path, {"do_sample": True, "temperature": 0.0}), {}).use_argmax


def test_sampling_defaults_environment_overrides(tmp_path):
    from zedinfer_b200.config import sampling_defaults
    d = _gen_folder(tmp_path, {"do_sample": True, "temperature": 0.6, "repetition_penalty": 1.05})
    assert sampling_defaults(d, {"ZEDINFER_FORCE_ARGMAX": "1"}).use_argmax
    assert not sampling_defaults(d, {"ZEDINFER_FORCE_ARGMAX": "0"}).use_argmax
    assert not sampling_defaults(d, {"ZEDINFER_FORCE_ARGMAX": ""}).use_argmax
    assert sampling_defaults(d, {"ZEDINFER_REPETITION_PENALTY": "1.3"}).repetition_penalty == 1.3
    assert sampling_defaults(d, {"ZEDINFER_REPETITION_PENALTY": "x"}).repetition_penalty == 1.05


def test_a_request_without_sampling_options_takes_the_engines_default():
    from zedinfer_b200.config import GenerationConfig
    default = GenerationConfig(use_argmax=False, temperature=0.6, top_k=20, top_p=0.9, seed=3)
    plain = GenerationConfig(max_new_tokens=5, ignore_eos=True)
    assert not plain.has_sampling_override
    r = plain.with_sampling_of(default)
    assert (r.max_new_tokens, r.ignore_eos, r.use_argmax, r.temperature, r.top_k, r.top_p, r.seed) == (5, True, False, 0.6, 20, 0.9, 3)
    own = GenerationConfig(max_new_tokens=5, use_argmax=False, temperature=1.3)
    assert own.has_sampling_override and own.with_sampling_of(default) is own
    greedy = GenerationConfig(max_new_tokens=5, has_sampling_override=True)      # insists on greedy
    assert greedy.with_sampling_of(default).use_argmax


# ---- command-line options (examples/ping.cpp:31-79, examples/serve.cpp:44-46, include/utils/logging_cli.hpp:11-38) ----
def test_command_line_options_map_to_the_scheduler_config(tmp_path, monkeypatch):
    import argparse
    import logging
    from zedinfer_b200.cli.common import add_engine_arguments, scheduler_config_from, setup_logging
    monkeypatch.delenv("ZEDINFER_KV_BLOCK_SIZE", raising=False)
    p = argparse.ArgumentParser()
    add_engine_arguments(p)
    a = p.parse_args(["/m"])
    sc = scheduler_config_from(a)
    assert (sc.max_batch_tokens, sc.max_batch_requests, sc.gpu_memory_utilization, sc.kv_block_size) == (2048, 64, 0.9, 16)
    assert sc.on_exhaust == "preempt" and sc.cuda_graphs and a.random_weights is None and a.dtype == "bfloat16"
    a = p.parse_args(["/m", "--max-batch-tokens", "512", "--max-batch-requests", "8", "--max-prefill-tokens", "128",
                      "--kv-block-size", "32", "--kv-pages", "100", "--max-seq-len", "4096", "--on-exhaust", "fail",
                      "--no-cuda-graphs", "--gpu-memory-utilization", "0.5", "--random-weights", "7", "--dtype", "float32",
                      "--log-level", "debug", "--log-file", str(tmp_path / "z.log"), "--no-log-to-console"])
    sc = scheduler_config_from(a)
    assert (sc.max_batch_tokens, sc.max_batch_requests, sc.max_prefill_tokens, sc.kv_block_size, sc.num_kv_pages,
            sc.max_seq_len, sc.on_exhaust, sc.cuda_graphs, sc.gpu_memory_utilization) == (512, 8, 128, 32, 100, 4096, "fail",
                                                                                           False, 0.5)
    sc.validate()
    log = setup_logging(a)
    log.debug("to the file only")
    assert log.level == logging.DEBUG and "to the file only" in (tmp_path / "z.log").read_text()
    for h in list(log.handlers):
        h.close()
        log.removeHandler(h)


def test_a_layer_names_its_parts_by_role():
    """Mixer and feed-forward are optional, further parts come under role names of their own, and no role is named twice."""
    from zedinfer_b200.config import LayerSpec, PartSpec
    norm = PartSpec("rmsnorm", {"size": 8, "eps": 1e-5})
    mix = PartSpec("attention", {})
    layer = LayerSpec("some_block", mix, None, {"norm1": norm}, {}, extra={"mixer2": ("mixer", mix), "gate_norm": ("norm", norm)})
    assert [(role, family) for role, family, _ in layer.part_specs()] == [
        ("mixer", "mixer"), ("norm1", "norm"), ("mixer2", "mixer"), ("gate_norm", "norm")]
    assert LayerSpec("b", None, None, {}, {}).part_specs() == ()
    for role in ("mixer", "norm1"):
        with pytest.raises(ValueError, match="repeats a role"):
            LayerSpec("b", mix, None, {"norm1": norm}, {}, extra={role: ("mixer", mix)}).part_specs()
