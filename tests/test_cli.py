"""The command line, run as a process: ``bin/vipera model-info | plan | random-weights`` and the
usage and exit-code cases on the CPU; ``generate`` on the GPU against the plain implementation.

What is checked follows the reference's contract (specs/001-vipera-rs-engine/contracts/cli.md:
19-87 for the commands, 186-231 for the exit codes; crates/vipera-errors/src/lib.rs:94-104) and
its own test of a continuation through the binary (bins/vipera/tests/llama_continuations.rs:27-101).
"""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

import helpers

VIPERA = os.path.join(helpers.ROOT, "bin", "vipera")
TOYS = os.path.join(helpers.ROOT, "tests", "toy_parts.py")

# Qwen2.5-32B's sizes: the shape whose batch of 64 at 8,192 tokens does not fit one 180 GB device.
SHAPE_32B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 64, "hidden_size": 5120,
    "num_attention_heads": 40, "num_key_value_heads": 8, "intermediate_size": 27648, "vocab_size": 152064,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 32768,
}


def vipera_process(*args, env_extra=None):
    """The command as a user runs it: a process of its own."""
    env = dict(os.environ)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, VIPERA, *args], capture_output=True, text=True, env=env, timeout=600)


class _Done:
    def __init__(self, returncode, stdout, stderr):
        self.returncode, self.stdout, self.stderr = returncode, stdout, stderr


def vipera(*args):
    """The same entry point called in this process (a process per case would spend most of the
    tests' time importing); the cases that need a process of their own use vipera_process."""
    import contextlib
    import io

    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200.cli import main

    out, err = io.StringIO(), io.StringIO()
    with contextlib.redirect_stdout(out), contextlib.redirect_stderr(err):
        code = main(list(args))
    return _Done(code, out.getvalue(), err.getvalue())


def config_folder(config) -> str:
    folder = tempfile.mkdtemp(prefix="vipera_cli_")
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config, handle)
    return folder


@pytest.fixture(scope="module")
def tiny_folder():
    source = config_folder(helpers.TINY_A)
    out = os.path.join(source, "model")
    done = vipera_process("random-weights", os.path.join(source, "config.json"), out, "--seed", "3", "--dtype", "float32")
    assert done.returncode == 0, done.stderr
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    return out


def test_random_weights_then_model_info(tiny_folder):
    done = vipera("model-info", tiny_folder, "--json")
    assert done.returncode == 0, done.stderr
    report = json.loads(done.stdout)
    a = helpers.TINY_A
    d = a["hidden_size"] // a["num_attention_heads"]
    q, kv = a["num_attention_heads"] * d, a["num_key_value_heads"] * d
    h, inter = a["hidden_size"], a["intermediate_size"]
    per_layer = h * q + 2 * h * kv + q + 2 * kv + q * h + 3 * h * inter + 2 * h
    assert report["parameter_count"] == a["num_hidden_layers"] * per_layer + a["vocab_size"] * h + h
    assert report["architecture"] == "Qwen2ForCausalLM" and report["layer_count"] == 2 and report["tied_output"]
    assert report["tensor_types"] == {"float32": report["tensor_count"]}
    assert report["kv_bytes_per_token_bf16"] == 2 * 2 * kv * 2
    plain = vipera("model-info", tiny_folder)
    assert plain.returncode == 0 and "parameter_count" in plain.stdout


def test_plan_feasible_and_infeasible(tiny_folder):
    done = vipera("plan", tiny_folder, "--ctx", "1024", "--batch", "4", "--json", "--device-bytes", str(10**9))
    assert done.returncode == 0, done.stderr
    report = json.loads(done.stdout)
    assert report["feasible"] and report["violations"] == []
    assert report["kv_bytes"] == 4 * 1024 * report["kv_bytes_per_token"]
    assert report["predicted_device_bytes"] == (report["weight_bytes"] + report["kv_bytes"]
                                                + report["workspace_bytes"] + report["reserve_bytes"])
    too_long = vipera("plan", tiny_folder, "--ctx", "100000", "--json")
    assert too_long.returncode == 3
    assert [v["constraint"] for v in json.loads(too_long.stdout)["violations"]] == ["context_limit"]
    too_small = vipera("plan", tiny_folder, "--ctx", "1024", "--device-bytes", "1000000")
    assert too_small.returncode == 3 and "device_memory" in too_small.stdout


def test_plan_refuses_batch_64_of_the_32b_shape_on_one_device():
    """64 requests of 8,192 tokens beside 65 GB of weights need more than 180 GB: the plan says so
    with exit code 3 (crates/vipera-core/src/planner.rs:276-430, bins/vipera/src/main.rs:186-251);
    eight such requests fit."""
    folder = config_folder(SHAPE_32B)
    flags = ["--ctx", "8192", "--dtype", "bfloat16", "--device-bytes", str(180 * 10**9), "--json"]
    wide = vipera("plan", folder, "--batch", "64", *flags)
    assert wide.returncode == 3, wide.stderr
    report = json.loads(wide.stdout)
    assert not report["feasible"] and report["violations"][0]["constraint"] == "device_memory"
    assert 64e9 < report["weight_bytes"] < 67e9
    assert report["kv_bytes"] == 64 * 8192 * 2 * 64 * 8 * 128 * 2       # 137 GB of keys and values
    assert report["predicted_device_bytes"] > 200e9
    narrow = vipera("plan", folder, "--batch", "8", *flags)
    assert narrow.returncode == 0 and json.loads(narrow.stdout)["feasible"]


def test_plan_and_model_info_ask_the_description_not_the_architecture():
    """Architectures registered from outside the package (one with a mixer that keeps a state of
    fixed size, one with other arrangements of a layer): plan and model-info need no change."""
    source = config_folder(dict(helpers.TINY_A, architectures=["ToyStateLM"]))
    env = {"VIPERA_PLUGINS": TOYS}
    done = vipera_process("plan", source, "--ctx", "512", "--batch", "3", "--dtype", "float32", "--json", env_extra=env)
    assert done.returncode == 0, done.stderr
    report = json.loads(done.stdout)
    a = helpers.TINY_A
    kv_width = a["num_key_value_heads"] * (a["hidden_size"] // a["num_attention_heads"])
    # layer 0 keeps a state of hidden + 1 floats per request, layer 1 keys and values
    assert report["kv_bytes_per_token"] == 2 * kv_width * 4
    assert report["kv_bytes"] == 3 * 512 * 2 * kv_width * 4 + 3 * (a["hidden_size"] + 1) * 4
    out = os.path.join(source, "model")
    arranged = config_folder(dict(helpers.TINY_A, architectures=["ToyArrangedLM"]))
    assert vipera_process("random-weights", os.path.join(arranged, "config.json"), out, env_extra=env).returncode == 0
    info = vipera_process("model-info", out, "--json", env_extra=env)
    assert info.returncode == 0, info.stderr
    report = json.loads(info.stdout)
    assert report["architecture"] == "ToyArrangedLM"
    # four norms in layer 0, one in layer 1, the final norm
    assert report["tensor_types"]["float32"] == 6
    unknown = vipera_process("model-info", out, "--json")   # without the plugin the architecture is not known
    assert unknown.returncode == 2 and "ToyArrangedLM" in unknown.stderr and "Qwen2ForCausalLM" in unknown.stderr


def test_usage_and_input_errors_have_their_exit_codes(tiny_folder):
    nothing = vipera_process()
    assert nothing.returncode == 1 and "usage: vipera" in nothing.stdout
    assert vipera("--help").returncode == 0
    unknown_command = vipera("serve", tiny_folder)
    assert unknown_command.returncode == 1 and 'unknown command "serve"' in unknown_command.stderr
    unknown_flag = vipera("generate", tiny_folder, "--prompt", "1 2", "--beam", "4")
    assert unknown_flag.returncode == 1 and 'unknown flag "--beam"' in unknown_flag.stderr
    assert "usage: vipera" in unknown_flag.stderr
    assert vipera("generate", tiny_folder).returncode == 1                          # no --prompt
    assert vipera("generate", tiny_folder, "--prompt").returncode == 1              # a flag without its value
    assert vipera("plan").returncode == 1
    words = vipera("generate", tiny_folder, "--prompt", "hello world")
    assert words.returncode == 2 and "token ids" in words.stderr and "Traceback" not in words.stderr
    assert vipera("generate", tiny_folder, "--prompt", "1 2", "--max-tokens", "many").returncode == 2
    assert vipera("generate", tiny_folder, "--prompt", "1 2", "--max-tokens", "0").returncode == 2
    assert vipera("generate", tiny_folder, "--prompt", "1 2", "--kv-type", "q8_0").returncode == 2
    missing = vipera("model-info", os.path.join(tiny_folder, "nowhere"))
    assert missing.returncode == 2 and "Traceback" not in missing.stderr
    broken = config_folder({"architectures": ["Qwen2ForCausalLM"], "hidden_size": 64})
    assert vipera("plan", broken).returncode == 2


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a device")
def test_generate_without_a_device_is_an_internal_error(tiny_folder):
    done = vipera_process("generate", tiny_folder, "--prompt", "1 2 3")
    assert done.returncode == 4
    assert done.stderr.startswith("vipera: internal:") and "Traceback" not in done.stderr
    assert len(done.stderr.strip().splitlines()) == 1


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_continues_like_the_plain_implementation(dtype):
    """A greedy continuation through the binary: every token is the plain model's best at its
    place, within the margin the dtype allows."""
    import numpy as np
    import plain_qwen2 as plain

    folder = helpers.model_folder("A", dtype)
    vocab = helpers.TINY_A["vocab_size"]
    prompt = helpers.random_tokens(vocab, 37, 5)
    done = vipera_process("generate", folder, "--prompt", " ".join(map(str, prompt)), "--max-tokens", "24",
                          "--dtype", dtype, "--json")
    assert done.returncode == 0, done.stderr
    report = json.loads(done.stdout.strip().splitlines()[-1])
    assert report["prompt_tokens"] == 37 and report["generated_tokens"] == 24 and report["finish"] == "length"
    tokens = report["tokens"]
    round_to = torch.bfloat16 if dtype == "bfloat16" else None
    logits = helpers.plain_logits(folder, prompt + tokens[:-1], round_to)
    margin = 1e-4 if dtype == "float32" else 2e-2
    for index, token in enumerate(tokens):
        row = logits[len(prompt) - 1 + index]
        assert row.max() - row[token] <= margin * np.abs(row).max(), f"token {index}"
    if dtype == "float32":
        config, weights = helpers.plain_model(folder)
        assert tokens == plain.greedy_continuation(config, weights, prompt, 24)
    streamed = vipera("generate", folder, "--prompt", ",".join(map(str, prompt)), "--max-tokens", "5", "--dtype", dtype)
    assert streamed.returncode == 0 and streamed.stdout.split() == [str(t) for t in tokens[:5]]
