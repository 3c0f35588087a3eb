"""The parts of bench.py's contract that need no GPU: what it answers for more than one GPU and for the
reference arm, its default arguments, and the arithmetic behind its fractions."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def run_bench(*args):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)
    lines = [ln for ln in p.stdout.splitlines() if ln.strip()]
    return p.returncode, lines


def test_more_than_one_gpu_is_one_line_and_exit_2():
    rc, lines = run_bench("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert rc == 2 and len(lines) == 1
    assert json.loads(lines[0])["n_gpus"] == 2


def test_reference_arm_says_unavailable_and_exits_0():
    rc, lines = run_bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert rc == 0 and len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_headline_shape_is_the_named_configuration():
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        named = json.load(f)["configs"][2]
    text = json.dumps(named).lower()
    assert "smollm2-1.7b" in text or "smollm2 1.7b" in text or "1.7b" in text
    s = bench.SHAPE
    assert (s["hidden_size"], s["num_hidden_layers"], s["num_attention_heads"], s["num_key_value_heads"],
            s["intermediate_size"], s["vocab_size"]) == (2048, 24, 32, 32, 8192, 49152)
    assert bench.CONTEXT == 4096 and bench.PREFILL_TOKENS == 2048


def test_weight_and_flop_counts():
    cfg = dict(bench.SHAPE)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    n = bench.model_numbers(cfg, 24)
    # 4 d^2 of attention and 3 d F of the feed-forward a layer; the tied head is read once a step
    assert n["layer_params"] == 4 * 2048 * 2048 + 3 * 2048 * 8192
    assert n["layer_params"] * 24 + n["head_params"] + n["norm_params"] == 1_711_376_384
    # a prompt of T tokens: 2 flops a weight and token, the head on one row, causal attention T^2 H hd a layer twice over
    T = 2048
    want = 2 * T * n["layer_params"] * 24 + 2 * n["head_params"] + 2 * T * T * 32 * 64 * 24
    assert bench.prefill_flops(cfg, 24, [T]) == want
    assert abs(want / 1e12 - 7.0096) < 1e-3
    # two prompts in one packed step do not attend to each other
    assert bench.prefill_flops(cfg, 24, [T, T]) == 2 * want


def test_prompt_length_distribution_argument():
    assert bench.parse_prompts("uniform:128-2048") == (128, 2048)
