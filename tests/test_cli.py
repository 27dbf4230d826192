"""Option parsing of the command line (no GPU); after crates/nncpu-cli/src/cli.rs:372-598."""
import pytest

from nncpu_b200.cli import main, parse_options, usage
from nncpu_b200.errors import InvalidArgument


def test_defaults_are_the_references():
    o = parse_options(["-m", "dir", "--tokens", "1 2 3"])
    assert (o.model, o.tokens, o.mode) == ("dir", "1 2 3", "generate")
    assert (o.temperature, o.top_k, o.top_p, o.min_p) == (0.7, 40, 0.95, 0.05)
    assert (o.n_predict, o.n_ctx, o.seed, o.dtype, o.kv_f32, o.perf, o.verbose) == (0, 0, 0, "bfloat16", False,
                                                                                   False, False)


def test_every_spelling():
    o = parse_options(["--model", "d", "--prompt", "hi", "--n_predict", "5", "--ctx_size", "99", "--top_k", "3",
                       "--top_p", "0.5", "--min_p", "0.1", "--temp", "0", "--seed", "7", "--kv-f32", "--perf", "-v"])
    assert (o.prompt, o.n_predict, o.n_ctx, o.top_k, o.top_p, o.min_p, o.temperature, o.seed) == \
        ("hi", 5, 99, 3, 0.5, 0.1, 0.0, 7)
    assert o.kv_f32 and o.perf and o.verbose
    o = parse_options(["-n", "8", "--n-predict", "9", "-c", "10", "--ctx-size", "11", "--top-k", "1", "--top-p", "1",
                       "--min-p", "0", "-s", "-5", "--fp32", "-b", "4"])
    assert (o.n_predict, o.n_ctx, o.top_k, o.seed, o.dtype, o.batch) == (9, 11, 1, 0, "float32", 4)
    assert parse_options(["--dtype", "bf16"]).dtype == "bfloat16"


def test_modes_take_their_arguments():
    o = parse_options(["--gen", "dir", "1 2 3", "16", "512", "--fp32"])
    assert o.mode == "gen" and o.args == ["dir", "1 2 3", "16", "512"] and o.dtype == "float32"
    assert parse_options(["--gen", "dir", "1 2"]).args == ["dir", "1 2"]
    assert parse_options(["--info", "dir"]).mode == "info"
    assert parse_options(["--random-weights", "c.json", "3", "out"]).args == ["c.json", "3", "out"]
    assert parse_options(["-h"]).mode == "help" and parse_options(["--version"]).mode == "version"


@pytest.mark.parametrize("argv", [["--gen", "dir"], ["-n"], ["-n", "x"], ["-n", "-1"], ["--temp", "-1"],
                                  ["--top-p", "1.5"], ["--min-p", "nan"], ["--dtype", "fp8"], ["--frobnicate"],
                                  ["-b", "0"]])
def test_refusals(argv):
    with pytest.raises(InvalidArgument):
        parse_options(argv)


def test_main_reports_errors(capsys):
    assert main(["--temp", "-1"]) == 1
    assert "InvalidArgument" in capsys.readouterr().err
    assert main(["--version"]) == 0
    assert main(["--help"]) == 0
    out = capsys.readouterr().out
    assert "--top-k N" in out and "--gen DIR" in out and usage().startswith("nncpu-b200")
    assert main(["-m", "x"]) == 1   # neither -p nor --tokens
