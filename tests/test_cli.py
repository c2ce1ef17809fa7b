"""The command line: option names and defaults of the reference's imp-cli, prompt parsing, and (on a
GPU) a run that prints the plain implementation's greedy tokens."""
import os
import subprocess
import sys

import pytest

from imp_b200.cli import build_parser, parse_prompt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "bin", "imp-cli")


def test_option_names_and_defaults_follow_the_reference():
    a = build_parser().parse_args(["--model", "m"])
    # tools/imp-cli/args.h:6-59
    assert (a.max_tokens, a.temperature, a.top_p, a.top_k, a.seed, a.min_p) == (256, 0.7, 0.9, 40, -1, 0.0)
    assert (a.repeat_penalty, a.frequency_penalty, a.presence_penalty, a.device) == (1.0, 0.0, 0.0, 0)
    assert (a.prefill_chunk_size, a.bench, a.bench_pp, a.bench_reps, a.no_cuda_graphs) == (0, False, 512, 3, False)
    b = build_parser().parse_args("--model m --prompt 1,2 --max-tokens 5 --temperature 0 --seed 7 --bench --bench-pp 64 "
                                  "--random-weights --weights-seed 3 --dtype fp32 --page-size 4 --kv-pages 10".split())
    assert b.bench and b.random_weights and b.dtype == "fp32" and b.kv_pages == 10 and b.page_size == 4
    with pytest.raises(SystemExit):
        build_parser().parse_args(["--prompt", "x"])           # --model is required
    with pytest.raises(SystemExit):
        build_parser().parse_args(["--model", "m", "--no-such-flag"])


def test_prompt_parsing():
    assert parse_prompt("5,17, 3", 100) == [5, 17, 3]
    assert parse_prompt("5 17 3", 100) == [5, 17, 3]
    assert parse_prompt("hi!", 256) == [104, 105, 33]            # any other text: its bytes
    with pytest.raises(SystemExit):
        parse_prompt("5,300", 256)
    with pytest.raises(SystemExit):
        parse_prompt("  ", 256)


@pytest.mark.gpu
def test_cli_generates_the_plain_tokens(model_folders):
    from plain.qwen3_plain import PlainModel
    folder, cd, page = model_folders["A"]
    want = PlainModel(folder).generate([5, 17, 3], 6)
    p = subprocess.run([sys.executable, CLI, "--model", folder, "--prompt", "5,17,3", "--max-tokens", "6",
                        "--temperature", "0", "--dtype", "fp32", "--page-size", str(page), "--kv-pages", "64",
                        "--max-seq-len", "128"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.split()] == want
    assert "pp " in p.stderr and "tg " in p.stderr and "tok/s" in p.stderr


@pytest.mark.gpu
def test_cli_random_weights_and_bench(model_folders, tmp_path):
    folder, cd, page = model_folders["B"]
    only_config = tmp_path / "cfg"
    only_config.mkdir()
    (only_config / "config.json").write_text(open(os.path.join(folder, "config.json")).read())
    base = [sys.executable, CLI, "--model", str(only_config), "--random-weights", "--weights-seed", "3",
            "--weights-std", "0.08", "--kv-pages", "64", "--max-seq-len", "256"]
    runs = [subprocess.run(base + ["--prompt", "1 2 3", "--max-tokens", "5", "--temperature", "0.9", "--seed", "11"],
                           capture_output=True, text=True, timeout=600) for _ in range(2)]
    assert all(r.returncode == 0 for r in runs), runs[0].stderr[-2000:]
    assert runs[0].stdout == runs[1].stdout and len(runs[0].stdout.split()) == 5     # same seeds, same tokens
    b = subprocess.run(base + ["--bench", "--bench-pp", "48", "--max-tokens", "8", "--bench-reps", "2", "--bench-batch", "2"],
                       capture_output=True, text=True, timeout=600)
    assert b.returncode == 0, b.stderr[-2000:]
    assert "pp    96 tokens" in b.stderr and "tg    16 tokens" in b.stderr
    bad = subprocess.run([sys.executable, CLI, "--model", str(tmp_path / "nowhere"), "--prompt", "1"],
                         capture_output=True, text=True, timeout=600)
    assert bad.returncode != 0 and "config.json" in bad.stderr
