"""Failure paths, made on the host or by a wait that runs out: a step that fails ends only its
own requests (crates/vipera-runtime/src/engine.rs:1625-1672), whatever kind of exception it was;
a bounded device wait that gives up is reported through the status word and leaves the device
usable.  No GPU fault is caused anywhere here."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _engine(**kwargs):
    from vipera_rs_b200 import Engine

    folder = helpers.model_folder("A", "float32")
    return folder, Engine(folder, dtype="float32", device=DEV, page_size=16, ctx=128, **kwargs)


@pytest.mark.parametrize("kind", ["internal", "other"])
def test_a_failing_step_ends_only_its_own_requests(kind):
    from test_engine_gpu import _check_greedy
    from vipera_rs_b200 import SamplingParams
    from vipera_rs_b200.errors import InternalError

    folder, engine = _engine(max_num_seqs=2, max_tokens_per_step=64, lookahead=False)
    vocab = helpers.CONFIGS["A"]["vocab_size"]
    prompts = [helpers.random_tokens(vocab, n, 40 + n) for n in (9, 14, 11)]
    ids = [engine.add_request(p, SamplingParams(max_new_tokens=6)) for p in prompts]
    real_run = engine.runner.run
    calls = {"n": 0}

    def failing_run(step):
        calls["n"] += 1
        if calls["n"] == 3:      # the two running requests are in their decode steps by then
            if kind == "internal":
                raise InternalError("made up: a kernel reported an error")
            raise ValueError("made up: a bug in a part")
        return real_run(step)

    engine.runner.run = failing_run
    finished = {}
    raised = 0
    while engine.has_work():
        try:
            report = engine.step()
        except InternalError as error:
            raised += 1
            assert "made up" in str(error)
            continue
        for generation in report.finished:
            finished[generation.request] = generation
    # the failed step's report was lost with the exception; its requests are gone from the scheduler
    assert raised == 1 and engine.failed == 2
    assert sorted(g.request for g in engine.failed_generations) == ids[:2]
    assert all(g.finish == "error" for g in engine.failed_generations)
    assert set(finished) == {ids[2]}                      # the request that waited was untouched ...
    assert finished[ids[2]].finish == "length" and len(finished[ids[2]].tokens) == 6
    _check_greedy(folder, prompts[2], finished[ids[2]].tokens, "float32")   # ... and its tokens are right
    assert engine.pools.audit() == "" and engine.stats()["sequences"] == 0
    assert engine.stats()["running"] == 0 and engine.stats()["waiting"] == 0
    # the engine goes on serving
    again = engine.generate([prompts[0]], SamplingParams(max_new_tokens=4))[0]
    _check_greedy(folder, prompts[0], again.tokens, "float32")


def test_a_refused_prompt_leaves_no_request_behind():
    from vipera_rs_b200 import SamplingParams
    from vipera_rs_b200.errors import ViperaError

    folder, engine = _engine(max_num_seqs=2)
    vocab = helpers.CONFIGS["A"]["vocab_size"]
    good = helpers.random_tokens(vocab, 10, 1)
    with pytest.raises(ViperaError):
        engine.generate([good, [1, 2, vocab + 5]], SamplingParams(max_new_tokens=4))
    with pytest.raises(ViperaError):
        engine.generate([good, helpers.random_tokens(vocab, 5000, 2)], SamplingParams(max_new_tokens=4))
    assert engine.stats()["waiting"] == 0 and engine.stats()["running"] == 0
    steps_before = engine.stats()["steps"]
    result = engine.generate([good], SamplingParams(max_new_tokens=4))[0]
    assert len(result.tokens) == 4
    assert engine.stats()["steps"] - steps_before <= 5    # nothing left over was run first
    assert engine.pools.audit() == ""


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200.errors import InternalError
    from vipera_rs_b200.kernels import ops

    device = torch.device(DEV)
    torch.manual_seed(0)
    a = (torch.randn(200, 256, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(384, 256, device=DEV) * 0.5).bfloat16()
    out = torch.empty(200, 384, device=DEV)
    ops.gemm_tc(a, w, epilogue=ops.EPI_STORE, out=out)      # builds the status word and proves the kernel works
    torch.cuda.synchronize()
    ops.check_kernel_status(device)                         # nothing to report
    ops.wait_probe(device, limit=3000)
    torch.cuda.synchronize()
    assert int(ops.kernel_status_word(device).item()) != 0
    with pytest.raises(InternalError) as info:
        ops.check_kernel_status(device)
    assert "gave up waiting" in str(info.value)
    assert int(ops.kernel_status_word(device).item()) == 0  # the word was cleared by the report
    ops.check_kernel_status(device)
    out.zero_()
    ops.gemm_tc(a, w, epilogue=ops.EPI_STORE, out=out)      # the next ordinary product is right
    torch.cuda.synchronize()
    want = a.double() @ w.double().T
    assert float((out.double() - want).abs().max() / want.abs().max()) < 1e-5
    ops.check_kernel_status(device)


def test_a_wait_that_runs_out_under_the_engine_fails_that_step_only():
    """The same through the engine: the status word is read with the step's tokens, the step's
    requests end with an error, the next request is served."""
    from test_engine_gpu import _check_greedy
    from vipera_rs_b200 import Engine, SamplingParams
    from vipera_rs_b200.errors import InternalError
    from vipera_rs_b200.kernels import ops

    folder = helpers.model_folder("A", "bfloat16")
    engine = Engine(folder, dtype="bfloat16", device=DEV, page_size=16, ctx=128, max_num_seqs=2, lookahead=False)
    vocab = helpers.CONFIGS["A"]["vocab_size"]
    prompt = helpers.random_tokens(vocab, 12, 3)
    engine.add_request(prompt, SamplingParams(max_new_tokens=5))
    engine.step()
    real_run = engine.runner.run

    def run_then_give_up(step):
        logits = real_run(step)
        ops.wait_probe(engine.model.device, limit=2000)
        return logits

    engine.runner.run = run_then_give_up
    with pytest.raises(InternalError):
        engine.step()
    engine.runner.run = real_run
    assert engine.failed == 1 and not engine.has_work()
    assert engine.pools.audit() == ""
    result = engine.generate([prompt], SamplingParams(max_new_tokens=5))[0]
    _check_greedy(folder, prompt, result.tokens, "bfloat16")
