"""Configuration parsing, the registry, safetensors I/O, weight errors and random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

import helpers
from nano_vllm_cpp_b200.config import (ConfigError, Qwen2MoeConfig, get_architecture, known_architectures,
                                       load_model_config)
from nano_vllm_cpp_b200.parts import Model
from nano_vllm_cpp_b200.weights import (SafetensorsFolder, SafetensorsError, save_safetensors, WeightsError,
                                        check_tensors, write_model_folder, RandomSource)

A = helpers.CASES["A"]["config"]
B = helpers.CASES["B"]["config"]


def test_parse_both_tiny_configs():
    a, b = Qwen2MoeConfig.from_dict(A), Qwen2MoeConfig.from_dict(B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert [a.layer_is_sparse(l) for l in range(2)] == [True, True]
    assert [a.layer_window(l) for l in range(2)] == [0, 0]
    assert a.norm_topk_prob and not a.tie_word_embeddings and a.rope_theta == 10000.0
    # B: step 2 makes layers 0 and 2 dense, mlp_only_layers names 2 as well; the window starts at layer 1
    assert [b.layer_is_sparse(l) for l in range(3)] == [False, True, False]
    assert [b.layer_window(l) for l in range(3)] == [0, 16, 16]
    assert b.tie_word_embeddings and not b.norm_topk_prob and b.rms_norm_eps == 1e-5


def test_head_dim_default_and_aliases():
    d = dict(A)
    del d["head_dim"]
    assert Qwen2MoeConfig.from_dict(d).head_dim == 16          # hidden_size / heads
    d = dict(A)
    d["num_local_experts"] = d.pop("num_experts")
    assert Qwen2MoeConfig.from_dict(d).num_experts == 8
    d = dict(A)
    d["norm_topk_probs"] = d.pop("norm_topk_prob")
    assert Qwen2MoeConfig.from_dict(d).norm_topk_prob is True
    d = dict(A)
    del d["num_key_value_heads"]
    assert Qwen2MoeConfig.from_dict(d).num_key_value_heads == 4


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
                                 "num_experts", "num_experts_per_tok", "moe_intermediate_size"])
def test_missing_required_key_is_named(key):
    d = dict(A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2MoeConfig.from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"hidden_size": "64"}, "hidden_size"), ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"), ({"num_experts_per_tok": 9}, "num_experts_per_tok"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"mlp_only_layers": [7]}, "mlp_only_layers"),
    ({"use_sliding_window": True, "sliding_window": 0}, "sliding_window"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"norm_topk_prob": 1}, "norm_topk_prob"), ({"decoder_sparse_step": 0}, "decoder_sparse_step"),
])
def test_bad_values_are_named(patch, word):
    d = dict(A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        Qwen2MoeConfig.from_dict(d)


def test_dense_layers_need_intermediate_size():
    d = dict(B)
    d["intermediate_size"] = 0
    with pytest.raises(ConfigError, match="intermediate_size"):
        Qwen2MoeConfig.from_dict(d)


def test_registry(tmp_path):
    assert "Qwen2MoeForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="Qwen2MoeForCausalLM"):
        get_architecture("NoSuchModel")
    (tmp_path / "config.json").write_text(json.dumps(A))
    arch, cfg = load_model_config(str(tmp_path))
    assert arch.name == "Qwen2MoeForCausalLM" and cfg.vocab_size == 256
    spec = arch.build_model(cfg)
    assert len(spec.layers) == 2 and spec.layers[0].feed_forward.kind == "sparse_moe_swiglu"
    b = get_architecture("Qwen2MoeForCausalLM").build_model(Qwen2MoeConfig.from_dict(B))
    assert [l.feed_forward.kind for l in b.layers] == ["dense_swiglu", "sparse_moe_swiglu", "dense_swiglu"]
    assert [l.mixer.params["window"] for l in b.layers] == [0, 16, 16]


def test_tensor_names_match_the_independent_table():
    """The names the model asks for are the names the golden script writes (HF naming)."""
    for case in ("A", "B"):
        cfg = helpers.CASES[case]["config"]
        spec = get_architecture("Qwen2MoeForCausalLM").build_model(Qwen2MoeConfig.from_dict(cfg))
        ours = {n: tuple(s.shape) for n, s in Model(spec).tensor_specs().items()}
        theirs = {n: tuple(shape) for n, shape, _ in helpers.make_golden.tensor_names(cfg)}
        assert ours == theirs


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.randn(2, 2, 2).to(torch.float16)}
    save_safetensors(str(tmp_path / "model.safetensors"), t, metadata={"x": 1})
    f = SafetensorsFolder(str(tmp_path))
    assert set(f.names()) == set(t)
    for n in t:
        got = f.load(n)
        assert got.dtype == t[n].dtype and got.shape == t[n].shape and torch.equal(got, t[n])
    # the independent reader of the plain implementation reads the same values
    save_safetensors(str(tmp_path / "model.safetensors"), {k: v for k, v in t.items() if k != "c"})
    (tmp_path / "config.json").write_text("{}")
    _, W = helpers.plain_model.read_folder(str(tmp_path))
    for n in ("a", "b", "d"):
        assert torch.equal(W[n], t[n].double())


def test_safetensors_bad_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x05")
    with pytest.raises(SafetensorsError, match="header"):
        SafetensorsFolder(str(tmp_path))
    import struct
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)       # data too short
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsFolder(str(tmp_path))
    (tmp_path / "empty").mkdir()
    with pytest.raises(SafetensorsError, match="no \\*.safetensors"):
        SafetensorsFolder(str(tmp_path / "empty"))


def test_weight_errors_list_everything(tmp_path):
    mdir = helpers.model_folder("A", str(tmp_path))
    f = SafetensorsFolder(mdir)
    tensors = {n: f.load(n) for n in f.names()}
    del tensors["model.layers.1.mlp.experts.3.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63, dtype=torch.bfloat16)
    tensors["model.layers.0.extra.weight"] = torch.zeros(2)
    bad = tmp_path / "bad"
    bad.mkdir()
    save_safetensors(str(bad / "model.safetensors"), tensors)
    spec = get_architecture("Qwen2MoeForCausalLM").build_model(Qwen2MoeConfig.from_dict(A))
    specs = Model(spec).tensor_specs()
    g = SafetensorsFolder(str(bad))
    with pytest.raises(WeightsError) as e:
        check_tensors(specs, {n: i.shape for n, i in g.tensors.items()})
    msg = str(e.value)
    assert "2 missing, 1 unexpected, 1 with a wrong shape" in msg
    assert "model.layers.1.mlp.experts.3.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.0.extra.weight" in msg
    assert "model.layers.0.self_attn.q_proj.weight: expected [64, 64], found [64, 63]" in msg


def test_untied_model_needs_lm_head_and_tied_model_rejects_it():
    a = Model(get_architecture("Qwen2MoeForCausalLM").build_model(Qwen2MoeConfig.from_dict(A))).tensor_specs()
    b = Model(get_architecture("Qwen2MoeForCausalLM").build_model(Qwen2MoeConfig.from_dict(B))).tensor_specs()
    assert "lm_head.weight" in a and "lm_head.weight" not in b


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    d1 = write_model_folder(B, str(tmp_path / "m1"), seed=5, std=0.05, norm_std=0.1)
    d2 = write_model_folder(B, str(tmp_path / "m2"), seed=5, std=0.05, norm_std=0.1)
    d3 = write_model_folder(B, str(tmp_path / "m3"), seed=6, std=0.05, norm_std=0.1)
    f1, f2, f3 = SafetensorsFolder(d1), SafetensorsFolder(d2), SafetensorsFolder(d3)
    assert json.load(open(os.path.join(d1, "config.json")))["num_experts"] == 6
    name = "model.layers.1.mlp.experts.2.down_proj.weight"
    assert torch.equal(f1.load(name), f2.load(name)) and not torch.equal(f1.load(name), f3.load(name))
    assert f1.load(name).dtype == torch.bfloat16
    w = f1.load("model.layers.0.input_layernorm.weight").float()
    assert abs(float(w.mean()) - 1.0) < 0.05 and 0.05 < float(w.std()) < 0.2
    big = f1.load("model.embed_tokens.weight").float()
    assert abs(float(big.std()) - 0.05) < 0.005
    # and the plain implementation can run it
    cfg, W = helpers.plain_model.read_folder(d1)
    out = helpers.plain_model.forward(cfg, W, [1, 2, 3])
    assert out.shape == (3, 384) and bool(torch.isfinite(out).all())


def test_random_source_is_order_independent():
    spec = get_architecture("Qwen2MoeForCausalLM").build_model(Qwen2MoeConfig.from_dict(A))
    specs = Model(spec).tensor_specs()
    s1 = RandomSource(specs, 3, 0.02, 0.0, "cpu", torch.bfloat16)
    s2 = RandomSource(specs, 3, 0.02, 0.0, "cpu", torch.bfloat16)
    names = list(specs)
    a = {n: s1.stored(n) for n in names}
    b = {n: s2.stored(n) for n in reversed(names)}
    assert all(torch.equal(a[n], b[n]) for n in names)


def _value_by_hand(seed, name, i, mean, std):
    """One value of the random-weights rule, restated with Python integers (64-bit wrap by masking)."""
    import hashlib
    import numpy as np
    M = (1 << 64) - 1

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)

    key = int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")
    c = (key + i * 0x9E3779B97F4A7C15) & M
    total = 0
    for h in (mix(c), mix(c ^ 0xD6E8FEB86659FD93), mix(c ^ 0xA0761D6478BD642F)):
        total += (h & 0xFFFF) + ((h >> 16) & 0xFFFF) + ((h >> 32) & 0xFFFF) + (h >> 48)
    z = np.float32(total - 393210) * np.float32(2.0 ** -16)
    return np.float32(mean) + z * np.float32(std)


def test_random_values_follow_the_stated_rule():
    """Every value is a function of (seed, name, element index); mean 0 and variance 1 before scaling."""
    import numpy as np
    from nano_vllm_cpp_b200.weights.random_values import host_values, tensor_key
    key = tensor_key(5, "model.layers.1.mlp.gate.weight")
    v = host_values(key, 5_000_003, 0.0, 1.0)             # more than one chunk of the host loop
    for i in (0, 1, 17, 4_194_303, 4_194_304, 5_000_002):
        assert v[i] == _value_by_hand(5, "model.layers.1.mlp.gate.weight", i, 0.0, 1.0)
    assert abs(float(v.mean())) < 2e-3 and abs(float(v.std()) - 1.0) < 2e-3
    assert abs(float(np.mean(v ** 4)) - 2.9) < 0.05        # twelve uniforms: kurtosis 3 - 0.1
    w = host_values(key, 1000, 1.0, 0.1)
    assert w[5] == _value_by_hand(5, "model.layers.1.mlp.gate.weight", 5, 1.0, 0.1)
    assert not np.array_equal(host_values(tensor_key(6, "model.layers.1.mlp.gate.weight"), 1000, 0.0, 1.0), v[:1000])
    assert not np.array_equal(host_values(tensor_key(5, "model.layers.0.mlp.gate.weight"), 1000, 0.0, 1.0), v[:1000])


def test_sampling_params_are_checked():
    from nano_vllm_cpp_b200 import SamplingParams
    SamplingParams(temperature=0.0, top_p=0.0, repetition_penalty=1.3, repetition_window=0).validate()
    for bad in (dict(temperature=-1.0), dict(max_tokens=0), dict(top_p=-0.1), dict(repetition_penalty=0.0),
                dict(repetition_penalty=float("nan")), dict(repetition_window=-1)):
        with pytest.raises(ValueError):
            SamplingParams(**bad).validate()
