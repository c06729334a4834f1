#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second and prefill tokens per
second on the Qwen2.5-1.5B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The default run decodes a batch of 8
requests, each with 2,048 tokens of history, and reports on ONE JSON line:

  value      decoded tokens per second, timed on the device (CUDA events around K steps of
             the engine's step function and its device sampler; token ids come from pinned
             host buffers, nothing is read back)
  e2e        the same through the public entry point ``Engine.step()``: scheduling, the
             host-to-device copy of the step's inputs and the device-to-host read of the
             sampled tokens included
  prefill    one prompt of 2,048 tokens: tokens per second, milliseconds, and the fraction
             of the bfloat16 tensor-core peak that its flops amount to
  roofline   bytes the decode step has to read (every weight once, the cache of the live
             requests) over its time, against the measured HBM copy bandwidth
  points     decode tokens per second at batch 1 and batch 64; prefill tokens per second for prompts
             of 128 and 512 tokens; milliseconds of a step of 8 decode tokens beside a 64-token portion
  mixed_7b   the Qwen2.5-7B shape under a mixed continuous batch through ``Engine.step()``
  shape_32b  the Qwen2.5-32B shape: decode at batch 1, 8 and the largest batch that fits, one prefill,
             and what the memory plan says about a batch of 64

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from the
figures measured earlier on the same pool (6.65 TB/s, 1.59 PFLOP/s).  Data are synthetic:
seeded random weights of the architecture's shapes and uniform random token ids.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_1P5B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 28, "hidden_size": 1536,
    "num_attention_heads": 12, "num_key_value_heads": 2, "intermediate_size": 8960, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "use_sliding_window": False, "sliding_window": 32768,
    "max_window_layers": 21,
}
QWEN25_0P5B = {   # head size 64
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 24, "hidden_size": 896,
    "num_attention_heads": 14, "num_key_value_heads": 2, "intermediate_size": 4864, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "use_sliding_window": False,
}
QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 28, "hidden_size": 3584,
    "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944, "vocab_size": 152064,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 32768, "use_sliding_window": False,
}
QWEN25_32B = {
    "architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 64, "hidden_size": 5120,
    "num_attention_heads": 40, "num_key_value_heads": 8, "intermediate_size": 27648, "vocab_size": 152064,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 32768, "use_sliding_window": False,
}
SHAPES = {"0.5b": ("Qwen2.5-0.5B shape", QWEN25_0P5B), "1.5b": ("Qwen2.5-1.5B shape", QWEN25_1P5B),
          "7b": ("Qwen2.5-7B shape", QWEN25_7B), "32b": ("Qwen2.5-32B shape", QWEN25_32B)}
FULL_LAYERS = 28
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as handle:
                data = json.load(handle)
            peaks = dict(FALLBACK_PEAKS)
            for key in peaks:
                if isinstance(data.get(key), (int, float)) and data[key] > 0:
                    peaks[key] = float(data[key])
            return peaks, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed work runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for parts in self.samples:
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons),
                "samples": len(clocks)}


def decode_bytes(config, layers, batch, history, element=2):
    """Bytes one decode step has to read: every weight it uses once (the embedding matrix only
    where it is also the output matrix), and the cache of the live requests at the mean history
    of the timed steps."""
    h, d = config["hidden_size"], config["hidden_size"] // config["num_attention_heads"]
    q, kv = config["num_attention_heads"] * d, config["num_key_value_heads"] * d
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * config["intermediate_size"]
    weights = (layers * per_layer + config["vocab_size"] * h) * element
    cache = batch * history * 2 * layers * kv * element
    return weights + cache


def prefill_flops(config, layers, tokens):
    h, d = config["hidden_size"], config["hidden_size"] // config["num_attention_heads"]
    q, kv = config["num_attention_heads"] * d, config["num_key_value_heads"] * d
    per_layer = h * (q + 2 * kv) + q * h + 3 * h * config["intermediate_size"]
    gemm = 2.0 * tokens * layers * per_layer + 2.0 * config["vocab_size"] * h
    attention = 2.0 * tokens * tokens * d * config["num_attention_heads"] * layers  # causal half of 4*T^2*d*heads
    return gemm + attention


class DecodeHarness:
    """`batch` requests with `history` tokens already in the cache (random keys and values,
    placed without running a prefill), decoded one token per step through the engine's
    runner and device sampler."""

    def __init__(self, model, batch, history, steps, page_size=16):
        import numpy as np
        import torch

        from vipera_rs_b200.cache import CachePools
        from vipera_rs_b200.engine import ModelRunner
        from vipera_rs_b200.sampling import DeviceSampler

        self.np, self.torch = np, torch
        self.model, self.batch, self.history = model, batch, history
        per_request = -(-(history + steps + 2) // page_size)
        self.pools = CachePools(model.cache_requests, page_size=page_size, num_pages=batch * per_request + 1,
                                num_state_slots=batch, dtype=model.dtype, device=model.device)
        for pool in self.pools.pool_tensors:
            pool.normal_(0.0, 0.5)
        self.runner = ModelRunner(model, self.pools, max_model_len=model.spec.max_position_embeddings)
        self.sampler_tokens = torch.empty(batch, dtype=torch.int32, device=model.device)
        self.manager = self.pools.manager
        self.requests = list(range(batch))
        for r in self.requests:
            self.manager.open(r)
            self.manager.reserve(r, history)
            self.manager.commit(r, history)
        self.position = history
        rng = np.random.default_rng(batch)
        self.token_stream = rng.integers(0, model.spec.vocab_size, size=(4096, batch), dtype=np.int32)
        self.cursor = 0

    def step(self):
        from vipera_rs_b200.engine import StepInput
        from vipera_rs_b200.kernels import ops

        np = self.np
        for r in self.requests:
            self.manager.reserve(r, self.position + 1)
        tokens = self.token_stream[self.cursor % 4096]
        self.cursor += 1
        step = StepInput(requests=self.requests, tokens=tokens, counts=[1] * self.batch,
                         pos0=[self.position] * self.batch, fresh=[0] * self.batch,
                         logit_rows=np.arange(self.batch, dtype=np.int32))
        logits = self.runner.run(step)
        ops.argmax(logits, self.sampler_tokens)
        for r in self.requests:
            self.manager.commit(r, self.position + 1)
        self.position += 1

    def timed(self, steps, warmup):
        torch = self.torch
        for _ in range(warmup):
            self.step()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first_position = self.position
        start.record()
        for _ in range(steps):
            self.step()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        mean_history = (first_position + self.position - 1) / 2.0 + 1
        return ms, mean_history

    def close(self):
        for r in self.requests:
            self.manager.close(r)


def measure_mixed_step(model, decodes, history, portion, repeats, warmup, page_size=16):
    """One step that carries `decodes` single tokens (each with `history` tokens behind it) and
    one prompt portion of `portion` tokens, as continuous batching makes them: milliseconds,
    median of `repeats`, device time of the step function and the device's greedy draw."""
    import numpy as np
    import torch

    from vipera_rs_b200.cache import CachePools
    from vipera_rs_b200.engine import ModelRunner, StepInput
    from vipera_rs_b200.kernels import ops

    per_request = -(-(history + warmup + repeats + 2) // page_size)
    pools = CachePools(model.cache_requests, page_size=page_size,
                       num_pages=decodes * per_request + -(-portion // page_size) + 1, num_state_slots=decodes + 1,
                       dtype=model.dtype, device=model.device)
    for pool in pools.pool_tensors:
        pool.normal_(0.0, 0.5)
    runner = ModelRunner(model, pools, max_model_len=model.spec.max_position_embeddings)
    manager = pools.manager
    for r in range(decodes):
        manager.open(r)
        manager.reserve(r, history)
        manager.commit(r, history)
    rng = np.random.default_rng(3)
    drawn = torch.empty(decodes + 1, dtype=torch.int32, device=model.device)
    times = []
    for index in range(warmup + repeats):
        position = history + index
        for r in range(decodes):
            manager.reserve(r, position + 1)
        manager.open(decodes)
        manager.reserve(decodes, portion)
        tokens = rng.integers(0, model.spec.vocab_size, size=decodes + portion, dtype=np.int32)
        step = StepInput(requests=list(range(decodes + 1)), tokens=tokens, counts=[1] * decodes + [portion],
                         pos0=[position] * decodes + [0], fresh=[0] * decodes + [1],
                         logit_rows=np.asarray(list(range(decodes)) + [decodes + portion - 1], dtype=np.int32))
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        logits = runner.run(step)
        ops.argmax(logits, drawn)
        stop.record()
        torch.cuda.synchronize()
        for r in range(decodes):
            manager.commit(r, position + 1)
        manager.close(decodes)
        if index >= warmup:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def measure_prefill(model, tokens, repeats, warmup, page_size=16):
    import numpy as np
    import torch

    from vipera_rs_b200.cache import CachePools
    from vipera_rs_b200.engine import ModelRunner, StepInput

    pools = CachePools(model.cache_requests, page_size=page_size, num_pages=-(-tokens // page_size) + 1,
                       num_state_slots=1, dtype=model.dtype, device=model.device)
    runner = ModelRunner(model, pools, max_model_len=model.spec.max_position_embeddings)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, model.spec.vocab_size, size=tokens, dtype=np.int32)
    times = []
    for index in range(warmup + repeats):
        pools.manager.open(0)
        pools.manager.reserve(0, tokens)
        step = StepInput(requests=[0], tokens=prompt, counts=[tokens], pos0=[0], fresh=[1],
                         logit_rows=np.asarray([tokens - 1], dtype=np.int32))
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.run(step)
        stop.record()
        torch.cuda.synchronize()
        pools.manager.close(0)
        if index >= warmup:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


def measure_e2e(model, batch, history, steps, warmup, page_size=16):
    """Through the public entry point: requests with `history`-token prompts are added and
    prefilled by the engine itself; then decode steps are timed on the host clock, each one
    scheduling, copying its inputs from pinned host memory, running, sampling and reading
    the sampled tokens back."""
    import numpy as np
    import torch

    from vipera_rs_b200 import Engine, SamplingParams

    per_request = -(-(history + steps + warmup + 8) // page_size)
    engine = Engine(model, page_size=page_size, num_pages=batch * per_request + 1, max_num_seqs=batch,
                    max_tokens_per_step=4096, max_portion=2048)
    rng = np.random.default_rng(1)
    params = SamplingParams(max_new_tokens=steps + warmup + 4, eos_ids=[])
    for _ in range(batch):
        engine.add_request(rng.integers(0, model.spec.vocab_size, size=history).tolist(), params)
    while True:  # prefill until every request decodes
        report = engine.step()
        if report.num_entries == batch and report.num_tokens == batch:
            break
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    started = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(engine.step().tokens)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    h2d = 4 * (8 * batch + 1 + batch * 256)  # packed int32 inputs of a decode step (tables 256 wide at most)
    d2h = 4 * (8 + 2 * batch)                 # token ids, row states and the kernels' status word, one copy
    return produced / elapsed, h2d, d2h


def release_memory():
    """Give back what finished harnesses held (runners and their captured graphs refer to one
    another, so the collector has to run before the allocator can let go)."""
    import gc

    import torch

    gc.collect()
    torch.cuda.empty_cache()


def measure_mixed(model, requests, prompt_range, new_tokens, max_portion, token_budget, passes=3, page_size=16):
    """The engine's normal mode: `requests` requests with prompt lengths uniform in
    `prompt_range`, all offered at once, prompts cut into portions of `max_portion` under a
    budget of `token_budget` tokens a step beside the running decodes, `new_tokens` tokens each,
    through ``Engine.step()`` on the host clock.  The first passes capture the graphs of the
    step sizes that occur (a buffer that grows in the first pass makes the graphs captured before
    it stale, so the second pass still captures some); the last pass is the one reported, with
    the number of graphs it still had to capture."""
    import numpy as np
    import torch

    from vipera_rs_b200 import Engine, SamplingParams

    rng = np.random.default_rng(7)
    lengths = rng.integers(prompt_range[0], prompt_range[1] + 1, size=requests)
    prompts = [rng.integers(0, model.spec.vocab_size, size=int(n)).tolist() for n in lengths]
    per_request = -(-(int(lengths.max()) + new_tokens + 1) // page_size)
    engine = Engine(model, page_size=page_size, num_pages=requests * per_request + 1, max_num_seqs=requests,
                    max_tokens_per_step=token_budget, max_portion=max_portion, prefix_cache=False)
    params = SamplingParams(max_new_tokens=new_tokens, eos_ids=[])
    report = {}
    for index in range(passes):
        before = dict(engine.totals, stage_micros=dict(engine.totals["stage_micros"]))
        captures_before = engine.runner.graph_captures
        for prompt in prompts:
            engine.add_request(prompt, params)
        torch.cuda.synchronize()
        started = time.perf_counter()
        generated = 0
        while engine.has_work():
            generated += len(engine.step().tokens)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - started
        totals = engine.totals
        steps = totals["steps"] - before["steps"]
        host = {stage: totals["stage_micros"][stage] - before["stage_micros"][stage] for stage in totals["stage_micros"]}
        prompt_tokens = int(lengths.sum())
        report = {
            "requests": requests, "prompt_tokens": prompt_tokens, "generated_tokens": generated,
            "prompt_min": int(prompt_range[0]), "prompt_max": int(prompt_range[1]), "new_tokens_each": new_tokens,
            "max_portion": max_portion, "token_budget": token_budget, "seconds": round(elapsed, 4),
            "tokens_per_s": round((prompt_tokens + generated) / elapsed, 1),
            "generated_tokens_per_s": round(generated / elapsed, 1),
            "steps": steps, "steps_with_portions": totals["steps_with_portions"] - before["steps_with_portions"],
            "tokens_per_step": round((totals["tokens"] - before["tokens"]) / max(steps, 1), 1),
            "ms_per_step": round(elapsed * 1e3 / max(steps, 1), 4),
            # the host's own work a step: scheduling, building and launching, bookkeeping (the
            # sample stage is mostly the wait for the device and is left out)
            "host_us_per_step": round((host["allocate"] + host["compute"] + host["complete"]) / max(steps, 1), 1),
            "host_us_allocate": round(host["allocate"] / max(steps, 1), 1),
            "host_us_compute": round(host["compute"] / max(steps, 1), 1),
            "host_us_complete": round(host["complete"] / max(steps, 1), 1),
            "wait_us_sample": round(host["sample"] / max(steps, 1), 1),
            "graph_step_share": round((totals["graph_steps"] - before["graph_steps"]) / max(steps, 1), 4),
            "graphs_captured_in_pass": engine.runner.graph_captures - captures_before,
            "timing": "host clock around Engine.step() until every request has ended",
        }
    del engine
    release_memory()
    return report


def measure_shape(name, config, layers, peaks, history, batches, steps, warmup, page_size=16, prefill_tokens=2048):
    """Decode at `batches` with `history` tokens of history and one prefill, for another shape."""
    import torch

    from vipera_rs_b200.engine import random_model

    full_layers = config["num_hidden_layers"]
    config = dict(config, num_hidden_layers=layers)
    model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    out = {"model": name, "layers": layers, "layers_full": full_layers, "seq_len": history, "dtype": "bf16"}
    for batch in batches:
        harness = DecodeHarness(model, batch, history, steps + warmup + 2, page_size=page_size)
        ms, mean_history = harness.timed(steps, warmup)
        harness.close()
        del harness
        release_memory()
        gbs = decode_bytes(config, layers, batch, mean_history) / (ms * 1e-3) / 1e9
        out[f"decode_b{batch}"] = round(batch * 1000.0 / ms, 1)
        out[f"decode_b{batch}_ms"] = round(ms, 4)
        out[f"decode_b{batch}_hbm_frac"] = round(gbs / peaks["hbm_gbs"], 4)
    ms = measure_prefill(model, prefill_tokens, repeats=3, warmup=2, page_size=page_size)
    out["prefill_tokens"] = prefill_tokens
    out["prefill_ms"] = round(ms, 3)
    out["prefill_tok_s"] = round(prefill_tokens * 1000.0 / ms, 1)
    out["prefill_frac"] = round(prefill_flops(config, layers, prefill_tokens) / (ms * 1e-3)
                                / (peaks["bf16_tflops_sustained"] * 1e12), 4)
    return out, model


def measure_32b(peaks, warmup, page_size):
    """The 32B shape: what the memory plan says about a batch of 64 at 8,192 tokens (it does not
    fit), decode at batch 1, 8 and the largest batch that fits, and one 2,048-token prefill."""
    import torch

    history = 8192
    refused = plan_report(QWEN25_32B, history + 256, 64)
    # the largest batch for the measurement is planned against what this device really has, less a
    # margin for the allocator
    usable = int(torch.cuda.get_device_properties(0).total_memory * 0.9)
    largest = 8
    for batch in range(8, 65, 8):
        if plan_report(QWEN25_32B, history + 256, batch, usable)["feasible"]:
            largest = batch
    out, model = measure_shape(SHAPES["32b"][0], QWEN25_32B, QWEN25_32B["num_hidden_layers"], peaks, history,
                               sorted({1, 8, largest}), steps=16, warmup=max(3, min(warmup, 4)), page_size=page_size)
    del model
    release_memory()
    out["largest_batch_that_fits"] = largest
    out["plan_b64_feasible"] = bool(refused["feasible"])
    out["plan_b64_needs_gb"] = round(refused["predicted_device_bytes"] / 1e9, 1)
    out["plan_device_gb"] = round(refused["device_bytes"] / 1e9, 1)
    return out


def plan_report(config, ctx, batch, device_bytes=180 * 10**9):
    """What `vipera plan` says about the shape at this context and batch (on one 180 GB device
    where nothing else is said)."""
    from vipera_rs_b200.config import architecture_of
    from vipera_rs_b200.engine import planner

    arch = architecture_of(config)
    return planner.plan_memory(arch.model_spec(arch.config_from_dict(config)), ctx, batch, "bfloat16", device_bytes)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--history", type=int, default=2048)
    parser.add_argument("--layers", type=int, default=FULL_LAYERS)
    parser.add_argument("--skip-points", action="store_true")
    parser.add_argument("--page-size", type=int, default=16, help="keys per cache page (the engine's default is 16)")
    parser.add_argument("--only", choices=["decode", "prefill", "mixed", "32b"], default=None,
                        help="run one part only and print a short line (for profiling a small case)")
    parser.add_argument("--config", choices=sorted(SHAPES), default="1.5b",
                        help="the shape the headline line is measured on (default: the 1.5B shape)")
    parser.add_argument("--prefill-tokens", type=int, default=2048)
    parser.add_argument("--skip-workloads", action="store_true",
                        help="leave out the 7B mixed workload and the 32B shape")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace that loads GGUF files; no cargo/rustc and no "
                          "GGUF model exist here, and pip cannot install it"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; bench.py measures --gpus 1 only",
                          "n_gpus": args.gpus}))
        return 2
    warmup = max(args.warmup, 3)

    import torch

    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200.engine import random_model

    peaks, peak_source = read_peaks()
    shape_name, shape = SHAPES[args.config]
    full_layers = shape["num_hidden_layers"]
    config = dict(shape)
    if args.layers == FULL_LAYERS and args.config != "1.5b":
        args.layers = full_layers
    config["num_hidden_layers"] = args.layers
    from vipera_rs_b200.kernels import ops

    model = random_model(config, seed=0, dtype="bfloat16", device="cuda:0")
    if args.only == "prefill":
        ms = measure_prefill(model, args.prefill_tokens, repeats=2, warmup=warmup, page_size=args.page_size)
        print(json.dumps({"only": "prefill", "layers": args.layers, "tokens": args.prefill_tokens, "ms": round(ms, 3),
                          "tok_s": round(args.prefill_tokens * 1000.0 / ms, 1)}))
        return 0
    if args.only == "mixed":
        print(json.dumps({"only": "mixed", "model": shape_name, "layers": args.layers,
                          **measure_mixed(model, 64, (128, 4096), 256, 512, 2048, page_size=args.page_size)}))
        return 0
    if args.only == "32b":
        del model
        release_memory()
        print(json.dumps({"only": "32b", **measure_32b(peaks, warmup, args.page_size)}))
        return 0
    if args.only == "decode":
        harness = DecodeHarness(model, args.batch, args.history, args.steps + 2 * warmup + 2, page_size=args.page_size)
        ms, _ = harness.timed(args.steps, warmup)
        print(json.dumps({"only": "decode", "layers": args.layers, "batch": args.batch, "ms_per_step": round(ms, 4)}))
        return 0
    sampler = ClockSampler()
    sampler.start()

    harness = DecodeHarness(model, args.batch, args.history, args.steps + warmup, page_size=args.page_size)
    harness.timed(2, warmup)  # graphs captured, buffers sized
    launches_before = ops.launches
    ms_per_step, mean_history = harness.timed(args.steps, warmup)
    timed_launches = ops.launches - launches_before
    harness.close()
    value = args.batch * 1000.0 / ms_per_step
    step_bytes = decode_bytes(config, args.layers, args.batch, mean_history)
    achieved_gbs = step_bytes / (ms_per_step * 1e-3) / 1e9

    points = {}
    if not args.skip_points:
        for batch in (1, 64):
            other = DecodeHarness(model, batch, args.history, 32 + warmup, page_size=args.page_size)
            ms, _ = other.timed(32, warmup)
            other.close()
            points[f"decode_b{batch}"] = round(batch * 1000.0 / ms, 1)
            del other
            release_memory()
        # steps as continuous batching makes them: short prompts whole, and a portion beside decodes
        for tokens in (128, 512):
            ms = measure_prefill(model, tokens, repeats=5, warmup=3, page_size=args.page_size)
            points[f"prefill_{tokens}"] = round(tokens * 1000.0 / ms, 1)
        points["step_8_decodes_and_64_token_portion_ms"] = round(
            measure_mixed_step(model, 8, args.history, 64, repeats=9, warmup=4, page_size=args.page_size), 4)
        release_memory()

    prefill_tokens = args.prefill_tokens
    prefill_ms = measure_prefill(model, prefill_tokens, repeats=5, warmup=3, page_size=args.page_size)
    flops = prefill_flops(config, args.layers, prefill_tokens)
    prefill_frac = flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12)

    e2e_value, h2d, d2h = measure_e2e(model, args.batch, args.history, args.steps, warmup, page_size=args.page_size)
    clocks = sampler.stop()

    # The engine's normal mode on the 7B shape and the 32B shape's decode and prefill: numbers of
    # their own beside the headline, each with the sizes it ran at.
    workloads = {}
    if args.config == "1.5b" and not args.skip_workloads:
        del model, harness
        release_memory()
        try:
            big = random_model(dict(QWEN25_7B), seed=1, dtype="bfloat16", device="cuda:0")
            workloads["mixed_7b"] = {"model": SHAPES["7b"][0], "layers": 28, "layers_full": 28,
                                     **measure_mixed(big, 64, (128, 4096), 256, 512, 2048, page_size=args.page_size)}
            del big
            release_memory()
            workloads["shape_32b"] = measure_32b(peaks, warmup, args.page_size)
        except Exception as error:  # the headline stands even where a larger shape does not fit
            workloads["error"] = f"{type(error).__name__}: {error}"

    line = {
        "metric": f"decode tok/s at batch {args.batch}, {args.history} tokens of history ({shape_name}); "
                  f"prefill tok/s at {prefill_tokens} tokens",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random token ids",
        "impl": "ours",
        "config": {
            "model": shape_name, "layers": args.layers, "layers_full": full_layers,
            "hidden": config["hidden_size"], "heads": config["num_attention_heads"],
            "kv_heads": config["num_key_value_heads"],
            "head_dim": config["hidden_size"] // config["num_attention_heads"],
            "intermediate": config["intermediate_size"], "vocab": config["vocab_size"],
            "tied_head": bool(config["tie_word_embeddings"]), "global_batch": args.batch, "seq_len": args.history,
            "new_tokens": args.steps, "page_size": args.page_size, "parallelism": "single GPU",
            "l2": "inputs larger than L2: every step reads all weights (GBs) against 126 MB",
            "peaks": peak_source,
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h,
                "overlap": "Engine.step() launches the step after while a step runs; both copies happen every step"},
        "gpu_launches": timed_launches,
        "prefill": {"value": round(prefill_tokens * 1000.0 / prefill_ms, 1), "tokens": prefill_tokens,
                    "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved_gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved_gbs / peaks["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }
    line.update(workloads)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
