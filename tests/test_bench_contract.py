"""What bench.py answers without a device: the reference arm (the reference cannot be installed
here) and a run on more than one GPU (this engine runs on one), and the bytes a decode step has
to read, which the roofline line divides by the step's time."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300)
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    return done.returncode, lines


def test_the_reference_arm_says_why_it_is_unavailable():
    code, lines = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert code == 0 and len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and record["unavailable"]


def test_more_than_one_gpu_is_one_line_and_exit_code_two():
    code, lines = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert code == 2 and len(lines) == 1
    assert json.loads(lines[0])["n_gpus"] == 2


def test_the_bytes_of_a_decode_step_count_every_weight_once_and_the_live_cache():
    sys.path.insert(0, ROOT)
    import bench

    config = dict(bench.QWEN25_1P5B)
    hidden, inter, vocab, layers = 1536, 8960, 151936, 28
    heads, kv_heads, d = 12, 2, 128
    per_layer = (hidden * (heads + 2 * kv_heads) * d + heads * d * hidden + 3 * hidden * inter) * 2
    weights = layers * per_layer + vocab * hidden * 2      # the tied matrix once
    cache = 8 * 2048 * layers * 2 * kv_heads * d * 2
    assert bench.decode_bytes(config, layers, batch=8, history=2048) == weights + cache
    # the line's own example: 3.09 GB of weights and 0.47 GB of cache at batch 8 and 2,048 keys
    assert abs(weights / 1e9 - 3.087) < 0.01 and abs(cache / 1e9 - 0.470) < 0.01
    # a prefill's flops: two per multiply-add of every matrix for every token, the vocabulary product
    # for the one wanted row, and the causal half of the scores and of the weighted sums
    elements = per_layer // 2
    expected = 2.0 * 2048 * layers * elements + 2.0 * vocab * hidden + 2.0 * 2048 * 2048 * d * heads * layers
    assert bench.prefill_flops(config, layers, 2048) == expected
    assert abs(expected / 1e12 - 5.73) < 0.01
