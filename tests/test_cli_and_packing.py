"""Command-line parsing, step packing, sampler options and the host restatement of the RNG (no GPU)."""
import numpy as np
import pytest

from rust_inference_b200 import SamplerConfig
from rust_inference_b200.cli import CliError, main, parse_args
from rust_inference_b200.engine.context import pack_step
from rust_inference_b200.sampling import rng


def test_flags_and_defaults_follow_the_reference(tmp_path):
    a = parse_args(["--model", str(tmp_path), "--prompt", "1,2,3"])
    # main.rs:65-70
    assert (a["max_tokens"], a["temperature"], a["top_k"], a["top_p"], a["seed"]) == (512, 0.8, 40, 0.95, 12345)
    assert a["max_seq_len"] is None and a["prompts"] == [[1, 2, 3]] and a["repetition_penalty"] == 1.1
    b = parse_args(["-m", str(tmp_path), "-p", "4 5", "-p", "6", "-n", "7", "-t", "0", "-k", "3", "--top-p", "0.5",
                    "-s", "9", "--max-seq-len", "64", "--dtype", "float32", "--stop-ids", "2,3"])
    assert b["prompts"] == [[4, 5], [6]] and b["max_tokens"] == 7 and b["temperature"] == 0.0
    assert (b["top_k"], b["top_p"], b["seed"], b["max_seq_len"]) == (3, 0.5, 9, 64)
    assert b["dtype"] == "float32" and b["stop_ids"] == [2, 3]


@pytest.mark.parametrize("argv, word", [
    (["--prompt", "1"], "--model is required"),
    (["--model"], "requires a value"),
    (["--model", "/nonexistent/x", "--prompt", "1"], "not found"),
    (["--model", ".", "--max-tokens", "many", "--prompt", "1"], "Invalid --max-tokens"),
    (["--model", ".", "--prompt", "1,a"], "Invalid token id"),
    (["--model", "."], "--prompt is required"),
    (["--model", ".", "--prompt", "1", "--frobnicate"], "Unknown argument"),
    (["--model", ".", "--prompt", "1", "--interactive"], "not available"),
])
def test_errors(argv, word):
    with pytest.raises(CliError, match=word):
        parse_args(argv)


def test_help_and_unknown_exit_codes(capsys):
    assert main(["--help"]) == 0                       # main.rs:160-163
    assert "Usage: gguf-infer" in capsys.readouterr().err
    assert main(["--bogus"]) == 1                      # main.rs:164-168
    assert "Unknown argument: --bogus" in capsys.readouterr().err


def test_prompt_file(tmp_path):
    f = tmp_path / "p.txt"
    f.write_text("1 2 3\n\n4,5\n")
    a = parse_args(["--model", str(tmp_path), "--prompt-file", str(f)])
    assert a["prompts"] == [[1, 2, 3], [4, 5]]


def test_sampler_config_defaults_are_the_reference():
    c = SamplerConfig()                                 # sampler.rs:37-48
    assert (c.temperature, c.top_k, c.top_p, c.repetition_penalty, c.repetition_window, c.seed) == \
        (0.8, 40, 0.95, 1.1, 64, 12345)
    assert c.uses_history and not c.greedy
    p = SamplerConfig.plain()
    assert p.greedy and not p.uses_history and p.top_k == 0 and p.top_p == 1.0
    with pytest.raises(ValueError):
        SamplerConfig(top_p=0.0)
    with pytest.raises(ValueError):
        SamplerConfig(repetition_penalty=0.0)


def test_pack_step_layout():
    meta, layout, sc = pack_step([10, 0, 64], [[7], [1, 2, 3], [9, 9]], [[0], [0, 2], []])

    def v(name):
        o, c = layout[name]
        return meta[o:o + c].tolist()

    assert v("token_ids") == [7, 1, 2, 3, 9, 9]
    assert v("token_pos") == [10, 0, 1, 2, 64, 65]           # positions continue from the cached length
    assert v("token_seq") == [0, 1, 1, 1, 2, 2]
    assert v("seq_start") == [10, 0, 64] and v("seq_len") == [11, 3, 66]
    assert v("cu_seqlens") == [0, 1, 4, 6]
    assert v("logit_rows") == [0, 1, 3]                      # order of sequences, then of places
    assert sc == {"n_tokens": 6, "n_seqs": 3, "n_logit_rows": 3, "max_new": 3, "max_len": 66, "all_single": False}
    assert pack_step([5, 6], [[1], [2]], [[0], [0]])[2]["all_single"] is True
    with pytest.raises(ValueError, match="outside"):
        pack_step([0], [[1, 2]], [[2]])
    assert meta.dtype == np.int32


def test_host_rng_is_a_uniform_in_open_closed_unit_interval():
    us = [rng.uniform(12345, s, c) for s in range(20) for c in range(50)]
    assert all(0.0 < u <= 1.0 for u in us)
    assert abs(sum(us) / len(us) - 0.5) < 0.03
    assert len(set(us)) > 990
    assert rng.uniform(1, 2, 3) == rng.uniform(1, 2, 3) != rng.uniform(1, 3, 2)
    assert all(u * 2 ** 24 == int(u * 2 ** 24) for u in us[:50])


def test_bench_contract_without_a_gpu():
    """`bench.py` for more than one GPU says so in one line and exits with 2; the reference arm prints
    its `unavailable` line and exits with 0; the benchmark model is configs[2] of BASELINE.json."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    bench = os.path.join(root, "bench.py")
    many = subprocess.run([sys.executable, bench, "--gpus", "2", "--steps", "2", "--warmup", "1"],
                          capture_output=True, text=True)
    assert many.returncode == 2 and len(many.stdout.strip().splitlines()) == 1
    ref = subprocess.run([sys.executable, bench, "--impl", "reference", "--gpus", "1"], capture_output=True, text=True)
    assert ref.returncode == 0
    line = json.loads(ref.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line
    sys.path.insert(0, root)
    import bench as bench_module
    m = bench_module.MODEL
    assert (m["num_hidden_layers"], m["hidden_size"], m["num_attention_heads"], m["num_key_value_heads"],
            m["head_dim"], m["intermediate_size"], m["vocab_size"]) == (28, 3584, 28, 4, 128, 18944, 152064)
    with open(os.path.join(root, "BASELINE.json")) as f:
        text = json.load(f)["configs"][2]
    for number in ("28 layers", "hidden 3584", "28 heads", "4 kv heads", "head_dim 128", "18944", "152064"):
        assert number in text


def test_flags_of_the_random_weights_mode(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text("{}")
    a = parse_args(["--random-config", str(cfg), "--weights-seed", "7", "--random-prompts", "3:5:9", "--slots", "2",
                    "--print-logits-topk", "4", "--dump-layer-stats", "--bench"])
    assert a["bench"] and a["random_config"] == str(cfg) and a["weights_seed"] == 7 and a["random_prompts"] == (3, 5, 9)
    assert a["slots"] == 2 and a["logits_topk"] == 4 and a["layer_stats"] and a["model"] is None
    for argv, word in [
        (["--random-config", str(cfg)], "--prompt is required"),
        (["--random-config", str(cfg), "--model", str(tmp_path), "--prompt", "1"], "exclude each other"),
        (["--random-config", str(tmp_path / "none.json"), "--prompt", "1"], "not found"),
        (["--model", str(tmp_path), "--random-prompts", "3:9:5"], "Invalid --random-prompts"),
        (["--model", str(tmp_path), "--random-prompts", "x"], "Invalid --random-prompts"),
        (["--model", str(tmp_path), "--prompt", "1", "--slots", "0"], "Invalid --slots"),
    ]:
        with pytest.raises(CliError, match=word):
            parse_args(argv)
