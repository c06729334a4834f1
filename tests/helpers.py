"""Shared by the tests: the tiny configurations, model folders, trace replay, comparison."""
from __future__ import annotations

import functools
import json
import os
import subprocess
import sys
import tempfile
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_qwen2 as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Three tiny configurations that differ in every size and option (B with windows in layers 1 and 2).
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 256,
    "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 704, "vocab_size": 512,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 2048, "use_sliding_window": False, "sliding_window": 4096,
    "max_window_layers": 2,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 384,
    "num_attention_heads": 3, "num_key_value_heads": 1, "intermediate_size": 1024, "vocab_size": 1003,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 4096, "use_sliding_window": True, "sliding_window": 80,
    "max_window_layers": 1,
}
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 240,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48, "intermediate_size": 336,
    "vocab_size": 777, "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 1024, "attention_bias": False,
}
# The two tiny configurations word for word as the baseline states them: A with 256 positions, B
# with full attention in all three layers (no window) and 512 positions.
TINY_A_STATED = dict(TINY_A, max_position_embeddings=256)
TINY_B_STATED = dict(TINY_B, use_sliding_window=False, max_position_embeddings=512)
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "A_stated": TINY_A_STATED, "B_stated": TINY_B_STATED}
SEEDS = {"A": 11, "B": 22, "C": 33, "A_stated": 11, "B_stated": 22}


@functools.lru_cache(maxsize=None)
def model_folder(name: str, store_dtype: str) -> str:
    """A model folder with random weights, made once per test session in a temporary place."""
    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200.engine import write_random_model

    path = tempfile.mkdtemp(prefix=f"vipera_tiny_{name}_{store_dtype}_")
    write_random_model(path, CONFIGS[name], SEEDS[name], store_dtype)
    return path


@functools.lru_cache(maxsize=None)
def plain_model(folder: str):
    return plain.read_config(folder), plain.read_weights(folder)


_PLAIN_CACHE: Dict[tuple, torch.Tensor] = {}


def plain_logits(folder: str, tokens: Sequence[int], round_to=None) -> np.ndarray:
    """Logits [len(tokens), vocab] of the plain implementation (float64 arithmetic)."""
    key = (folder, tuple(tokens), round_to)
    if key not in _PLAIN_CACHE:
        config, weights = plain_model(folder)
        _PLAIN_CACHE[key] = plain.forward(config, weights, list(tokens), dtype=torch.float64,
                                          round_to=round_to).numpy()
    return _PLAIN_CACHE[key]


def random_tokens(vocab: int, count: int, seed: int) -> List[int]:
    rng = np.random.default_rng(seed)
    return [int(x) for x in rng.integers(0, vocab, size=count)]


def run_trace(folder: str, dtype: str, steps: List[dict], max_tokens: int, page_size: int = 64,
              env_extra=None, timeout: int = 900, max_live: int = 8) -> Dict[int, np.ndarray]:
    """Replay ``steps`` with bin/trace_run as a user would (a process of its own) and return
    the logits files it wrote, by step."""
    vocab = json.load(open(os.path.join(folder, "config.json")))["vocab_size"]
    out_dir = tempfile.mkdtemp(prefix="vipera_trace_out_")
    text = "".join(json.dumps(step) + "\n" for step in steps)
    env = dict(os.environ)
    env["VIPERA_POISON_CACHE"] = "1"
    env.update(env_extra or {})
    command = [sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
               "--max-tokens", str(max_tokens), "--page-size", str(page_size), "--max-live", str(max_live)]
    result = subprocess.run(command, input=text, capture_output=True, text=True, env=env, timeout=timeout)
    if result.returncode != 0:
        raise AssertionError(f"trace_run exited with {result.returncode}\nstdout:\n{result.stdout[-2000:]}\n"
                             f"stderr:\n{result.stderr[-4000:]}")
    done = [line for line in result.stdout.splitlines() if line.startswith("done ")]
    assert [int(line.split()[1]) for line in done] == [step["step"] for step in steps], result.stdout[-2000:]
    outputs = {}
    for step in steps:
        wanted = sum(len(entry.get("want", [])) for entry in step["entries"])
        path = os.path.join(out_dir, f"{step['step']}.f32")
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == wanted * vocab, f"step {step['step']}: {data.size} values for {wanted} rows"
            outputs[step["step"]] = data.reshape(wanted, vocab)
        else:
            assert not os.path.exists(path)
    return outputs


class TraceBuilder:
    """Builds a trace and remembers, for every wanted row, which request and position it is."""

    def __init__(self):
        self.steps: List[dict] = []
        self.expect: Dict[int, List[tuple]] = {}  # step -> [(request name, position)]
        self._done: Dict[str, int] = {}

    def step(self, entries, end=()):
        """entries: [(name, tokens, want places)]"""
        number = len(self.steps)
        record = {"step": number, "entries": [], "end": list(end)}
        expect = []
        for name, tokens, want in entries:
            first = self._done.get(name, 0)
            record["entries"].append({"id": name, "tokens": list(tokens), "want": list(want)})
            expect.extend((name, first + place) for place in want)
            self._done[name] = first + len(tokens)
        for name in end:
            self._done.pop(name, None)
        self.steps.append(record)
        if expect:
            self.expect[number] = expect
        return number


def compare(outputs, builder: TraceBuilder, reference: Dict[str, np.ndarray], tolerance: float, what: str):
    """Hold every emitted row to the plain implementation's row at the same request and
    position: max |difference| <= tolerance * max |plain logit| of that request."""
    worst = 0.0
    for number, expect in builder.expect.items():
        rows = outputs[number]
        for index, (name, position) in enumerate(expect):
            want = reference[name][position]
            got = rows[index]
            assert np.isfinite(got).all(), f"{what}: step {number} request {name} position {position}: not finite"
            scale = float(np.abs(reference[name]).max())
            error = float(np.abs(got - want).max()) / scale
            worst = max(worst, error)
            assert error <= tolerance, (
                f"{what}: step {number}, request {name}, position {position}: "
                f"relative error {error:.3e} exceeds {tolerance:.1e}")
    return worst
