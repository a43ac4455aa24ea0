"""Configuration parsing, the architecture registry, safetensors reading and
the loader's errors.  No GPU."""

import json
import os

import pytest
import torch

import plain_model as pm
from tiny_configs import ALL, TINY_A, TINY_B, TINY_C
from ullm_b200.config import (ConfigError, EngineConfig, Qwen3Config, load_model_spec, register_architecture,
                              resolve_architecture)
from ullm_b200.parts import DecoderModel
from ullm_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights, save_tensors,
                               write_random_model)


def test_qwen3_config_reads_its_keys():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 80, 9, 3)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 176, 331)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings
    assert c.dtype == "float32" and c.max_position_embeddings == 256


def test_qwen3_config_defaults_follow_the_reference():
    d = {k: TINY_A[k] for k in ("architectures", "num_hidden_layers", "hidden_size", "num_attention_heads",
                                "num_key_value_heads", "intermediate_size", "vocab_size")}
    c = Qwen3Config.from_dict(d)
    assert c.head_dim == 64 // 4  # hidden_size // num_attention_heads
    assert c.rope_theta == 1000000.0  # getattr default in ullm/models/qwen3.py:144
    assert c.rms_norm_eps == 1e-6 and c.attention_bias is False
    assert c.dtype == "float16"  # ullm/core/model_runner.py:38-51: neither "dtype" nor "torch_dtype" -> float16
    assert Qwen3Config.from_dict(dict(d, dtype="bfloat16")).dtype == "bfloat16"  # "dtype" wins over "torch_dtype"
    # transformers 5 keeps theta under rope_parameters
    c2 = Qwen3Config.from_dict(dict(d, rope_parameters={"rope_theta": 5000.0, "rope_type": "default"}))
    assert c2.rope_theta == 5000.0


@pytest.mark.parametrize("patch,match", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "SiLU"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope scaling"),
    ({"torch_dtype": "int8"}, "dtype"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
])
def test_bad_configs_are_refused(patch, match):
    d = dict(TINY_A)
    d.update(patch)
    if patch.get("hidden_size", 0) is None:
        del d["hidden_size"]
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict(d)


def test_registry():
    assert resolve_architecture(TINY_A).name == "Qwen3ForCausalLM"
    with pytest.raises(ValueError, match="not supported.*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    _, spec = load_model_spec(TINY_C)
    assert [l.mixer.args["window"] for l in spec.layers] == [None, None, 24, 24]
    assert spec.layers[0].mixer.args["qkv_bias"] is True
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3]


def test_model_spec_carries_every_size(tmp_path):
    _, spec = load_model_spec(TINY_B)
    m = DecoderModel(spec)
    decls = m.all_decls()
    assert {n: tuple(d.shape) for n, d in decls.items()} == pm.tensor_shapes(TINY_B)
    _, specA = load_model_spec(TINY_A)
    assert "lm_head.weight" not in DecoderModel(specA).all_decls()  # tied


def _write(tmp_path, cfg, w, name="m"):
    d = tmp_path / name
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    save_tensors(str(d / "model.safetensors"), w)
    return str(d)


def _model(cfg, untie=False):
    _, spec = load_model_spec(cfg)
    m = DecoderModel(spec, untie_head=untie)
    m.allocate("cpu", torch.float32)
    return m


def test_loader_places_fused_rows_and_keeps_norms_32bit(tmp_path):
    cfg, init, _ = ALL["C"]
    w = {n: t.to(torch.bfloat16) for n, t in pm.random_weights(cfg, **init).items()}
    d = _write(tmp_path, cfg, w)
    _, spec = load_model_spec(cfg)
    m = DecoderModel(spec)
    m.allocate("cpu", torch.bfloat16)
    seen = load_weights(m, d)
    assert set(seen) == set(w)
    att = m.blocks[1].mixer
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    assert torch.equal(att.w_qkv[:q], w["model.layers.1.self_attn.q_proj.weight"])
    assert torch.equal(att.w_qkv[q:q + kv], w["model.layers.1.self_attn.k_proj.weight"])
    assert torch.equal(att.w_qkv[q + kv:], w["model.layers.1.self_attn.v_proj.weight"])
    assert torch.equal(att.b_qkv[:q], w["model.layers.1.self_attn.q_proj.bias"])
    ff = m.blocks[2].feed_forward
    I = cfg["intermediate_size"]
    assert torch.equal(ff.w_gate_up[:I], w["model.layers.2.mlp.gate_proj.weight"])
    assert torch.equal(ff.w_gate_up[I:], w["model.layers.2.mlp.up_proj.weight"])
    assert att.w_qkv.dtype == torch.bfloat16
    assert m.final_norm.tensors["weight"].dtype == torch.float32
    assert att.q_norm.tensors["weight"].dtype == torch.float32
    assert torch.equal(m.final_norm.tensors["weight"], w["model.norm.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg, init, _ = ALL["B"]
    w = pm.random_weights(cfg, **init)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    w["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(10, 80)
    w["model.embed_tokens.weight"] = torch.zeros(300, 80)
    d = _write(tmp_path, cfg, w)
    with pytest.raises(WeightError) as ei:
        load_weights(_model(cfg), d)
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert {n for n, _, _ in e.wrong_shape} == {"model.layers.2.self_attn.k_proj.weight", "model.embed_tokens.weight"}
    msg = str(e)
    for piece in ("missing (2)", "unexpected (1)", "wrong shape (2)", "file (300, 80) != model (331, 80)"):
        assert piece in msg


def test_tied_head(tmp_path):
    cfg, init, _ = ALL["A"]
    w = pm.random_weights(cfg, **init)
    d = _write(tmp_path, cfg, w)
    m = _model(cfg)
    load_weights(m, d)
    assert m.head.weight().data_ptr() == m.embedding.tensors["weight"].data_ptr()
    # an untied config without lm_head.weight is an error that names it
    cfgu = dict(cfg, tie_word_embeddings=False)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(_model(cfgu), _write(tmp_path, cfgu, w, "u"))
    # a tied config whose file carries lm_head.weight uses that tensor
    w2 = dict(w)
    w2["lm_head.weight"] = w["model.embed_tokens.weight"] * 2
    m2 = _model(cfg, untie=True)
    load_weights(m2, _write(tmp_path, cfg, w2, "t"))
    assert torch.equal(m2.head.weight(), w2["lm_head.weight"])


def test_truncated_and_corrupt_files(tmp_path):
    cfg, init, _ = ALL["A"]
    d = _write(tmp_path, cfg, pm.random_weights(cfg, **init))
    path = os.path.join(d, "model.safetensors")
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[: len(raw) - 100])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(path)
    open(path, "wb").write(b"\x05\x00\x00\x00\x00\x00\x00\x00hello")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(path)
    os.remove(path)
    with pytest.raises(FileNotFoundError):
        load_weights(_model(cfg), d)


def test_random_model_folder_is_seeded_and_loadable(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_B, seed=5, std=0.03, norm_std=0.1)
    b = write_random_model(str(tmp_path / "b"), TINY_B, seed=5, std=0.03, norm_std=0.1)
    c = write_random_model(str(tmp_path / "c"), TINY_B, seed=6, std=0.03, norm_std=0.1)
    ra = open(os.path.join(a, "model.safetensors"), "rb").read()
    assert ra == open(os.path.join(b, "model.safetensors"), "rb").read()
    assert ra != open(os.path.join(c, "model.safetensors"), "rb").read()
    f = SafetensorsFile(os.path.join(a, "model.safetensors"))
    assert {n: f.shape(n) for n in f.names()} == pm.tensor_shapes(TINY_B)
    t = f.get("model.layers.0.mlp.down_proj.weight")
    assert abs(t.std().item() - 0.03) < 0.003
    n = f.get("model.norm.weight")
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.2
    m = _model(TINY_B)
    load_weights(m, a)
    assert json.load(open(os.path.join(a, "config.json")))["vocab_size"] == 331
    # the written folder round-trips through the plain implementation
    w = {k: f.get(k).clone() for k in f.names()}
    assert pm.forward_logits([1, 2, 3], w, TINY_B).shape == (3, 331)


def test_engine_config_names_and_checks(tmp_path):
    d = _write(tmp_path, TINY_A, pm.random_weights(TINY_A, seed=0, std=0.02, norm_std=0.05))
    ec = EngineConfig(model=d, gpu_memory_utilization=0.8, max_bs=4, tp_size=1, pp_size=1, context_len=64)
    assert ec.model_config["hidden_size"] == 64 and ec.enforce_eager is False and ec.nccl_port == 29500
    with pytest.raises(ValueError, match="one GPU"):
        EngineConfig(model=d, tp_size=2)
    (tmp_path / "m" / "generation_config.json").write_text(json.dumps({"temperature": 0.6, "top_k": 20, "top_p": 0.95}))
    sp = EngineConfig(model=d).get_default_sampling_params()
    assert (sp.temperature, sp.top_k, sp.top_p, sp.min_p) == (0.6, 20, 0.95, 0.0)
    import argparse

    ap = argparse.ArgumentParser()
    EngineConfig.add_cli_args(ap)
    ns = ap.parse_args(["--model", d, "--max-bs", "7", "--context-len", "99", "--enforce-eager"])
    ec2 = EngineConfig.from_args(ns)
    assert (ec2.max_bs, ec2.context_len, ec2.enforce_eager, ec2.gpu_memory_utilization) == (7, 99, True, 0.9)


def test_a_new_architecture_needs_one_registration():
    from ullm_b200.config import ARCHITECTURES, qwen3_model_spec

    def spec_twice(cfg):
        s = qwen3_model_spec(cfg)
        s.architecture = "TwiceForCausalLM"
        from ullm_b200.config import ScheduleEntry

        s.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(0, cache_of=0)]
        return s

    register_architecture("TwiceForCausalLM", Qwen3Config.from_dict, spec_twice)
    try:
        _, spec = load_model_spec(dict(TINY_A, architectures=["TwiceForCausalLM"]))
        m = DecoderModel(spec)
        needs = m.cache_needs()
        assert len(needs) == 4 and needs[3][2] == 0 and needs[2][2] is None
    finally:
        ARCHITECTURES.pop("TwiceForCausalLM")
