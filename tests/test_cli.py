"""The command line's parsing and defaults (no device needed)."""
import pytest

from torchless_rs_b200 import cli


def test_default_max_tokens_rule():
    assert cli.resolve_max_tokens(None, 32768) == 8192      # max_seq_len / 4
    assert cli.resolve_max_tokens(None, 4096) == 2048       # clamped from below at 2048
    assert cli.resolve_max_tokens(None, 2048) == 1024
    assert cli.resolve_max_tokens(None, 10 ** 6) == 32768
    assert cli.resolve_max_tokens(7, 4096) == 7


def test_options_and_positionals():
    o = cli.parse_args(["--max-tokens", "5", "--temperature", "0", "--top-k", "40", "--top-p", "0.9",
                        "--seed", "3", "--dtype", "float32", "--stop", "2,7", "--debug", "dir", "1 2 3"])
    assert (o["max_tokens"], o["temperature"], o["top_k"], o["top_p"]) == (5, 0.0, 40, 0.9)
    assert o["seed"] == 3 and o["dtype"] == "float32" and o["stop"] == (2, 7) and o["debug"]
    assert o["positional"] == ["dir", "1 2 3"]
    assert cli.parse_args(["dir"])["temperature"] == 0.7      # the reference's default
    assert cli.parse_args(["--backend", "cuda", "dir"])["positional"] == ["dir"]
    o = cli.parse_args(["--random-weights", "--weights-seed", "9", "--save-weights", "dir"])
    assert o["random_weights"] and o["weights_seed"] == 9 and o["save_weights"] and o["positional"] == ["dir"]
    assert not cli.parse_args(["dir"])["random_weights"]


def test_prompts_are_token_ids():
    assert cli.parse_prompts("1 5 9") == [[1, 5, 9]]
    assert cli.parse_prompts("1,5,9 ; 1 7;") == [[1, 5, 9], [1, 7]]
    with pytest.raises(ValueError, match="token ids"):
        cli.parse_prompts("hello world")


def test_errors_exit_with_one(capsys):
    assert cli.main(["--no-such-flag", "dir"]) == 1
    assert "unknown option '--no-such-flag'" in capsys.readouterr().err
    assert cli.main(["--chat", "dir"]) == 1
    assert "not available" in capsys.readouterr().err
    assert cli.main(["--backend", "metal", "dir"]) == 1
    assert cli.main(["--max-tokens"]) == 1
    assert cli.main(["--max-tokens", "x", "dir"]) == 1
    assert cli.main([]) == 1
    assert "Usage" in capsys.readouterr().err
    assert cli.main(["--help"]) == 0
    assert cli.main(["/nonexistent/model"]) == 1
