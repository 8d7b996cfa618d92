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
