"""The command line's own decisions, which need no GPU: usage, help, refused front ends, bad values
(exit codes of src/main.cpp:432-438: 1 usage, 2 error)."""
from nano_vllm_cpp_b200 import cli


def test_no_arguments_is_a_usage_error(capsys):
    assert cli.main([]) == 1
    assert "Usage: nanovllm" in capsys.readouterr().err


def test_help(capsys):
    assert cli.main(["--help"]) == 0
    err = capsys.readouterr().err
    for word in ("--tokens", "--max-tokens", "--temperature", "--max-model-len", "--bench", "--num-seqs", "--num-kv-blocks"):
        assert word in err


def test_front_ends_that_are_not_built_are_refused(capsys):
    for flag in ("--chat", "--server"):
        assert cli.main(["model", flag]) == 2
        assert flag in capsys.readouterr().err


def test_bad_values_and_missing_model(capsys):
    assert cli.main(["model", "--max-tokens", "many"]) == 1
    assert "bad option value" in capsys.readouterr().err
    assert cli.main(["model", "--tokens", "1,x,3"]) == 1
    assert cli.main(["--bench"]) == 1                       # no model folder
    assert cli.main(["model", "a prompt", "one word too many"]) == 1


def test_a_text_prompt_is_refused_before_anything_is_loaded(capsys):
    assert cli.main(["model", "Hello"]) == 2
    assert "--tokens" in capsys.readouterr().err


def test_token_list():
    assert cli.parse_ids("1,2, 3,") == [1, 2, 3]


def test_generation_config_gives_defaults_that_options_override(tmp_path, monkeypatch):
    import json
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"temperature": 0.25, "top_p": 0.8, "max_new_tokens": 7, "eos_token_id": [5, 6]}))
    assert cli.generation_defaults(str(tmp_path)) == {"temperature": 0.25, "top_p": 0.8, "max_tokens": 7}
    seen = {}
    monkeypatch.setattr(cli, "_run", lambda opt: seen.update(opt) or 0)
    assert cli.main([str(tmp_path), "--tokens", "1,2", "--top-p", "0.5"]) == 0
    assert (seen["temperature"], seen["top_p"], seen["max_tokens"]) == (0.25, 0.5, 7)
    # a broken or absent file gives nothing and never fails
    (tmp_path / "generation_config.json").write_text("{ not json")
    assert cli.generation_defaults(str(tmp_path)) == {}
    assert cli.generation_defaults(str(tmp_path / "nowhere")) == {}
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": "hot", "max_new_tokens": 0}))
    assert cli.generation_defaults(str(tmp_path)) == {}


def test_config_option_runs_random_weights_without_a_folder(tmp_path, monkeypatch):
    """``--config <json>`` stands for a model folder: the run gets a temporary folder whose config.json is the file
    and draws its weights from ``--seed``."""
    import json
    import os
    cfg = tmp_path / "tiny.json"
    cfg.write_text(json.dumps({"architectures": ["Qwen2MoeForCausalLM"], "hidden_size": 64}))
    seen = {}

    def fake_run(opt):
        seen.update(opt)
        with open(os.path.join(opt["model_dir"], "config.json")) as f:
            seen["config_json"] = json.load(f)
        return 0

    monkeypatch.setattr(cli, "_run", fake_run)
    assert cli.main(["--config", str(cfg), "--seed", "7", "--tokens", "1,2", "--dtype", "fp32"]) == 0
    assert seen["random_weights"] is True and seen["seed"] == 7 and seen["dtype"] == "fp32"
    assert seen["config_json"]["hidden_size"] == 64
    assert not os.path.exists(seen["model_dir"])            # the temporary folder is gone afterwards
    assert cli.main(["--config", str(tmp_path / "absent.json"), "--tokens", "1"]) == 2


def test_dtype_spellings():
    from nano_vllm_cpp_b200.config import EngineConfig
    import pytest
    for given, want in (("bf16", "bfloat16"), ("fp32", "float32"), ("bfloat16", "bfloat16"), ("float32", "float32")):
        c = EngineConfig(dtype=given)
        c.validate()
        assert c.dtype == want
    with pytest.raises(ValueError, match="dtype"):
        EngineConfig(dtype="half").validate()
