"""The public entry point: requests in, tokens out, by continuous batching.

The surface follows the reference's ``Engine`` (crates/vipera-runtime/src/engine.rs):
``admit``+``enqueue`` become ``add_request`` (engine.rs:396, 606), ``step`` returns what the
step produced (engine.rs:671-765), ``generate`` loops ``step`` until its requests end
(engine.rs:563-591), ``cancel`` frees a request's pages at once (engine.rs:1199-1206) and
``stats`` reports the cache (engine.rs:94-110, 380-390).  A finished request's record
carries the reference's ``Generation`` fields (engine.rs:62-82).
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..build import runtime_module
from ..cache import CachePools
from ..errors import InternalError, InvalidArgumentError, ViperaError
from ..kernels import ops
from ..sampling import DeviceSampler, SamplingParams
from .loader import load_model
from .runner import ModelRunner, StepInput


@dataclass
class Generation:
    """How a request ended."""

    request: int
    tokens: List[int]            # generated tokens, the end token included
    finish: str                  # "stop" | "length" | "cancelled" | "error"
    prompt_tokens: int
    processed_tokens: int        # tokens run through the model, recomputation included
    preemptions: int
    reused_tokens: int = 0       # prompt tokens whose keys and values an earlier request had computed
    # Host microseconds of the steps the request took part in, by stage (the reference's stage
    # names, crates/vipera-runtime/src/pipeline.rs:17-72): allocate = scheduling and page
    # reservation, compute = building and launching the step, sample = drawing and waiting for
    # the tokens, complete = bookkeeping after the step.  A step's time counts for each of its requests.
    stage_micros: Dict[str, int] = field(default_factory=dict)
    # Where the request asked for them (``SamplingParams.logprobs``): the log-probability of every
    # generated token under the distribution it was drawn from, and the most likely tokens there
    # with theirs, best first (crates/vipera-sampler/src/lib.rs:302-378).
    logprobs: Optional[List[float]] = None
    top_logprobs: Optional[List[List[tuple]]] = None

    def to_json(self) -> str:
        """One line in the shape of the reference's request log (pipeline.rs:234-271)."""
        import json

        return json.dumps({"event": "generation", "sequence": self.request, "prompt_tokens": self.prompt_tokens,
                           "reused_tokens": self.reused_tokens, "generated_tokens": len(self.tokens),
                           "finish": self.finish, "total_micros": sum(self.stage_micros.values()),
                           "stage_micros": self.stage_micros})


@dataclass
class StepReport:
    tokens: List[tuple] = field(default_factory=list)        # (request, token) drawn in this step
    finished: List[Generation] = field(default_factory=list)
    preempted: List[int] = field(default_factory=list)
    num_tokens: int = 0                                       # tokens the step ran
    num_entries: int = 0
    graph: bool = False                                       # the step replayed a captured graph
    stage_micros: Dict[str, int] = field(default_factory=dict)  # host time of the step by stage


class _RowsAhead:
    """What the sampler needs to know about the rows of a step launched ahead: the rows of
    the step before (the same requests in the same order) with the uniform draws the scheduler
    will hand out next."""

    any_penalty = False
    all_greedy = False

    def __init__(self, plan, uniforms: np.ndarray):
        self.row_temperature, self.row_top_k = plan.row_temperature, plan.row_top_k
        self.row_top_p, self.row_min_p = plan.row_top_p, plan.row_min_p
        self.row_uniform = uniforms

    def same_as(self, plan) -> bool:
        return (not plan.any_penalty and np.array_equal(plan.row_temperature, self.row_temperature)
                and np.array_equal(plan.row_top_k, self.row_top_k) and np.array_equal(plan.row_top_p, self.row_top_p)
                and np.array_equal(plan.row_min_p, self.row_min_p) and np.array_equal(plan.row_uniform, self.row_uniform))


class _Ahead:
    """A decode step launched before the plan that asks for it exists."""

    __slots__ = ("requests", "positions", "logits", "drawn", "rows")

    def __init__(self, requests, positions, logits, drawn, rows):
        self.requests, self.positions, self.logits, self.drawn = list(requests), positions, logits, drawn
        self.rows = rows  # None: every row greedy

    def serves(self, plan) -> bool:
        """Whether `plan` is the step that was launched: the same requests, one token each at
        the positions foreseen, every row drawn the way it was drawn."""
        count = len(self.requests)
        if not (plan.num_entries == count and plan.num_tokens == count and plan.num_rows == count
                and plan.requests == self.requests and np.array_equal(plan.starts, self.positions)):
            return False
        if self.rows is None:
            return plan.all_greedy and not plan.any_penalty
        return self.rows.same_as(plan)


class Engine:
    """One model on one GPU, a paged cache and a scheduler.

    ``model`` is a folder (config.json and model.safetensors) or a built ``DecoderModel``.
    ``prefix_cache``: full pages of prompts stay known after their request ends and are shared
    with requests that begin with the same tokens (the reference's prefix cache,
    crates/vipera-runtime/src/engine.rs:432-491, which copies them); they are given up, least
    recently used first, when pages are needed.
    ``lookahead``: while a step of greedy decoding runs, the step after it is launched already
    where the scheduler can foresee it, so that the host's share of a step (scheduling, input
    copies, the launch, reading tokens back) hides behind the device's.
    ``ctx`` is the context length each of ``max_num_seqs`` requests can reach with the
    pages allocated (default: the smaller of the model's limit and 2048, as the reference's
    ``--ctx``, bins/vipera/src/main.rs:655-663); ``num_pages`` overrides that sizing.
    """

    def __init__(self, model, dtype="bfloat16", device="cuda:0", *, page_size: int = 16,
                 num_pages: Optional[int] = None, ctx: Optional[int] = None, max_num_seqs: int = 4,
                 max_tokens_per_step: int = 2048, max_portion: Optional[int] = None,
                 max_model_len: Optional[int] = None, decode_graphs: bool = True, prefix_cache: bool = True,
                 lookahead: bool = True):
        if isinstance(model, str):
            model = load_model(model, dtype, device)
        self.model = model
        limit = model.spec.max_position_embeddings
        self.max_model_len = min(limit, max_model_len) if max_model_len else limit
        if ctx is None:
            ctx = min(self.max_model_len, 2048)
        if num_pages is None:
            num_pages = max_num_seqs * ((ctx + page_size - 1) // page_size)
        self.pools = CachePools(model.cache_requests, page_size=page_size, num_pages=num_pages,
                                num_state_slots=max_num_seqs, dtype=model.dtype, device=model.device,
                                reuse_prefixes=prefix_cache)
        self.runner = ModelRunner(model, self.pools, max_model_len=self.max_model_len)
        self.runner.decode_graphs = decode_graphs
        runtime = runtime_module()
        self.scheduler = runtime.Scheduler(self.pools.manager, int(max_num_seqs), int(max_tokens_per_step),
                                           int(max_portion or max_tokens_per_step), int(self.max_model_len),
                                           bool(prefix_cache))
        self.sampler = DeviceSampler(model.device)
        self.default_eos = tuple(getattr(getattr(model, "config", None), "eos_token_ids", ()) or ())
        self._next_id = 0
        self.generations = 0
        self.failed = 0
        # The records of requests that ended with a failed step (the step's report is lost with
        # the exception that step() raises); the caller may read and clear the list.
        self.failed_generations: List[Generation] = []
        # A step launched ahead may be dropped and run again; keys and values are then written
        # twice with the same numbers, but a state of fixed size that a mixer updates in place
        # would move twice.  Models with such state decode step by step.
        self.lookahead = bool(lookahead) and not self.pools.states
        self._ahead: Optional[_Ahead] = None
        self.steps_ahead = 0          # steps launched before their plan existed ...
        self.steps_ahead_dropped = 0  # ... and those of them whose plan turned out otherwise
        self.totals = {"steps": 0, "tokens": 0, "entries": 0, "graph_steps": 0, "steps_with_portions": 0,
                       "stage_micros": {"allocate": 0, "compute": 0, "sample": 0, "complete": 0}}
        self._request_micros: Dict[int, Dict[str, int]] = {}
        self._logprobs: Dict[int, tuple] = {}   # request -> (top n, temperature, logprobs so far, top lists so far)
        # VIPERA_PROFILE_STEP=1: a line per step on stderr (what ran, how, the host's time by stage),
        # and a line per finished request in the shape of the reference's request log.
        self.profile_steps = os.environ.get("VIPERA_PROFILE_STEP", "0") not in ("", "0")
        self.kernel_profile = None
        if self.profile_steps:
            # the split of a step's device time by class of kernel needs steps launched kernel by
            # kernel, one at a time
            self.kernel_profile = ops.profile = ops.KernelProfile()
            self.runner.decode_graphs = self.runner.step_graphs = False
            self.lookahead = False

    # ------------------------------------------------------------------------------
    def add_request(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[int] = None) -> int:
        params = params or SamplingParams()
        if request_id is None:
            request_id = self._next_id
        self._next_id = max(self._next_id, request_id + 1)
        prompt = [int(t) for t in prompt_ids]
        vocab = self.model.spec.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise InvalidArgumentError(f"prompt holds a token id outside the vocabulary of {vocab}")
        if params.logprobs is not None and not 0 <= int(params.logprobs) <= 64:
            raise InvalidArgumentError("logprobs must be between 0 and 64 (the number of most likely tokens reported)")
        self.scheduler.add(int(request_id), prompt, params.to_native(self.default_eos))
        if params.logprobs is not None:
            self._logprobs[int(request_id)] = (int(params.logprobs), float(params.temperature), [], [])
        return int(request_id)

    def cancel(self, request_id: int) -> None:
        self.scheduler.cancel(int(request_id))

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> StepReport:
        clock = time.perf_counter
        t0 = clock()
        plan = self.scheduler.schedule()
        t1 = clock()
        report = StepReport(preempted=list(plan.preempted), num_tokens=int(plan.num_tokens),
                            num_entries=int(plan.num_entries))
        ahead, self._ahead = self._ahead, None
        t2 = t3 = t1
        if plan.empty:
            outcome = self.scheduler.complete(plan, [])
        else:
            replays = self.runner.graph_replays
            try:
                drawn = logits = None
                if ahead is not None and ahead.serves(plan):
                    # this step was launched while the one before still ran
                    drawn, logits = ahead.drawn, ahead.logits
                    ahead = None
                    replays -= 1
                else:
                    step = StepInput(requests=plan.requests, tokens=plan.tokens, counts=plan.counts, pos0=plan.starts,
                                     fresh=plan.fresh, logit_rows=plan.row_token_index)
                    if self.kernel_profile is not None:
                        self.kernel_profile.begin()
                    logits = self.runner.run(step)
                    if logits is not None:
                        drawn = self.sampler.launch(logits, plan)
                t2 = clock()
                if drawn is not None:
                    if self.lookahead:
                        self._ahead = self._launch_ahead(plan)
                    # also reads the kernels' status word
                    sampled = self.sampler.collect(drawn, logits, plan, logits_intact=self._ahead is None)
                    if self._logprobs:
                        self._record_logprobs(plan, logits, sampled)
                else:
                    sampled = []
                    torch.cuda.current_stream().synchronize()
                    ops.check_kernel_status(self.model.device)
                t3 = clock()
                outcome = self.scheduler.complete(plan, sampled)
                if self._ahead is not None and outcome["finished"]:
                    # a request ended on the token just read: the step launched ahead is not the next one
                    self._ahead = None
                    self.steps_ahead_dropped += 1
            except BaseException as error:
                # Whatever went wrong, the plan's requests do not stay half-run: they end with
                # reason "error" and give their pages back, the others go on
                # (crates/vipera-runtime/src/engine.rs:1625-1672).  A fault of the engine itself
                # is raised as it is; anything else is raised too, after the same clean-up.
                self._ahead = None
                outcome = self.scheduler.fail(plan)
                self.failed += len(outcome["finished"])
                self._collect(report, outcome)
                self.failed_generations.extend(report.finished)
                if isinstance(error, ViperaError) or not isinstance(error, Exception):
                    raise
                raise InternalError(f"a step failed: {type(error).__name__}: {error}") from error
            report.graph = self.runner.graph_replays > replays
        if ahead is not None:
            self.steps_ahead_dropped += 1
        t4 = clock()
        stages = {"allocate": int((t1 - t0) * 1e6), "compute": int((t2 - t1) * 1e6),
                  "sample": int((t3 - t2) * 1e6), "complete": int((t4 - t3) * 1e6)}
        report.stage_micros = stages
        self._account(plan, report, stages)
        self._collect(report, outcome)
        return report

    def _account(self, plan, report: StepReport, stages: Dict[str, int]) -> None:
        """Add the step to the engine's counters and to the stage times of its requests."""
        if plan.empty:
            return
        totals = self.totals
        totals["steps"] += 1
        totals["tokens"] += report.num_tokens
        totals["entries"] += report.num_entries
        totals["graph_steps"] += 1 if report.graph else 0
        if report.num_tokens > report.num_entries:
            totals["steps_with_portions"] += 1
        for stage, micros in stages.items():
            totals["stage_micros"][stage] += micros
        for request in plan.requests:
            mine = self._request_micros.setdefault(int(request), dict.fromkeys(stages, 0))
            for stage, micros in stages.items():
                mine[stage] += micros
        if self.profile_steps:
            kind = "chunk" if report.num_tokens > report.num_entries else "decode"
            if self.kernel_profile is not None:
                self.kernel_profile.end(kind)
                print(self.kernel_profile.line(kind), file=sys.stderr, flush=True)
            print(f"STEP {totals['steps']} {kind} entries {report.num_entries} tokens {report.num_tokens} "
                  f"{'graph' if report.graph else 'eager'} host_us " +
                  " ".join(f"{stage} {micros}" for stage, micros in stages.items()), file=sys.stderr, flush=True)

    def _launch_ahead(self, plan) -> Optional["_Ahead"]:
        """Where the scheduler can tell what the next step is before this one's tokens are
        read (everybody decodes, greedily or with a top-k the device draws alone, without
        penalties, and nobody can end but by an end token), launch it now:
        its input tokens pass from this step's draw to its embedding on the device.  The next
        call of step() takes it over if its plan is the one foreseen, and drops it otherwise;
        a dropped step has only written keys and values that the step run in its stead writes
        again, or that belong to requests that ended."""
        if not self.scheduler.plan_ahead(plan, ops.SAMPLER_MAX_TOP_K):
            return None
        if self._logprobs and any(int(r) in self._logprobs for r in plan.row_requests):
            return None   # the log-probabilities are read from this step's logits after its tokens
        requests = plan.requests
        positions = plan.starts + 1
        count = len(requests)
        logits = self.runner.run_ahead(requests, positions, self.sampler.device_tokens(count))
        if logits is None:
            return None
        self.steps_ahead += 1
        rows = None if plan.all_greedy else _RowsAhead(plan, self.scheduler.peek_uniforms(plan))
        return _Ahead(requests, positions, logits, self.sampler.launch(logits, rows), rows)

    def _record_logprobs(self, plan, logits: torch.Tensor, sampled) -> None:
        """For the rows of requests that asked: the log-probability of the token just drawn and
        the most likely tokens, computed on the device from the step's logits (penalties are
        already applied to them)."""
        wanted = [(row, int(request)) for row, request in enumerate(plan.row_requests) if int(request) in self._logprobs]
        if not wanted:
            return
        top_n = max(self._logprobs[request][0] for _, request in wanted)
        device = logits.device
        rows = torch.tensor([row for row, _ in wanted], dtype=torch.int32, device=device)
        tokens = torch.tensor([int(sampled[row]) for row, _ in wanted], dtype=torch.int32, device=device)
        temperature = torch.tensor([self._logprobs[request][1] for _, request in wanted], dtype=torch.float32, device=device)
        chosen, top_ids, top_values = ops.logprobs(logits, rows, tokens, temperature, top_n)
        chosen, top_ids, top_values = chosen.tolist(), top_ids.tolist(), top_values.tolist()
        for index, (_, request) in enumerate(wanted):
            count, _, values, tops = self._logprobs[request]
            values.append(chosen[index])
            tops.append([(int(i), float(v)) for i, v in zip(top_ids[index][:count], top_values[index][:count]) if i >= 0])

    def _collect(self, report: StepReport, outcome: dict) -> None:
        report.tokens.extend((int(r), int(t)) for r, t in outcome["tokens"])
        for item in outcome["finished"]:
            generation = Generation(
                request=int(item["request"]), tokens=[int(t) for t in item["tokens"]], finish=item["reason"],
                prompt_tokens=int(item["prompt_tokens"]), processed_tokens=int(item["processed_tokens"]),
                preemptions=int(item["preemptions"]), reused_tokens=int(item["reused_tokens"]),
                stage_micros=self._request_micros.pop(int(item["request"]), {}))
            asked = self._logprobs.pop(generation.request, None)
            if asked is not None:
                generation.logprobs, generation.top_logprobs = asked[2][:len(generation.tokens)], asked[3][:len(generation.tokens)]
            report.finished.append(generation)
            self.generations += 1
            if self.profile_steps:
                print(generation.to_json(), file=sys.stderr, flush=True)

    def generate(self, prompts: Sequence[Sequence[int]], params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token=None) -> List[Generation]:
        """Run prompts (lists of token ids) to their ends; results in the order given."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise InvalidArgumentError("one SamplingParams is needed for each prompt, or one for all")
        ids = []
        try:
            for prompt, p in zip(prompts, params):
                ids.append(self.add_request(prompt, p))
        except BaseException:
            # A prompt that is refused must not leave the ones before it waiting in the
            # scheduler for a later call to run: they are cancelled (they hold no pages yet; the
            # next step reports them as cancelled).
            for request in ids:
                self.cancel(request)
            raise
        results: Dict[int, Generation] = {}
        while len(results) < len(ids):
            if not self.has_work():
                raise InternalError("the scheduler has no work left but requests are unfinished")
            report = self.step()
            if on_token is not None:
                for request, token in report.tokens:
                    on_token(request, token)
            for generation in report.finished:
                if generation.request in ids:
                    results[generation.request] = generation
        return [results[i] for i in ids]

    def stats(self) -> dict:
        manager = self.pools.manager
        groups = [manager.stats(g) for g in range(manager.num_groups)]
        totals = self.totals
        steps = max(totals["steps"], 1)
        return {
            "steps": totals["steps"],
            "steps_with_portions": totals["steps_with_portions"],
            "graph_steps": totals["graph_steps"],
            "tokens_per_step": totals["tokens"] / steps,
            "entries_per_step": totals["entries"] / steps,
            "host_micros_per_step": {stage: micros / steps for stage, micros in totals["stage_micros"].items()},
            "steps_ahead": self.steps_ahead,
            "steps_ahead_dropped": self.steps_ahead_dropped,
            "sequences": len(manager.open_requests()),
            "waiting": self.scheduler.num_waiting,
            "running": self.scheduler.num_running,
            "kv_used_pages": sum(g["used_pages"] for g in groups),
            "kv_free_pages": sum(g["free_pages"] for g in groups),
            "kv_kept_pages": sum(g["kept_pages"] for g in groups),
            "kv_total_bytes": self.pools.bytes(),
            "groups": groups,
            "generations": self.generations,
            "failed": self.failed,
        }
