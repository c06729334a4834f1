"""The public entry point: requests in, tokens out, by continuous batching.

The surface follows the reference's ``Engine`` (crates/vipera-runtime/src/engine.rs):
``admit``+``enqueue`` become ``add_request`` (engine.rs:396, 606), ``step`` returns what the
step produced (engine.rs:671-765), ``generate`` loops ``step`` until its requests end
(engine.rs:563-591), ``cancel`` frees a request's pages at once (engine.rs:1199-1206) and
``stats`` reports the cache (engine.rs:94-110, 380-390).  A finished request's record
carries the reference's ``Generation`` fields (engine.rs:62-82).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..build import runtime_module
from ..cache import CachePools
from ..errors import InternalError, InvalidArgumentError
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


@dataclass
class StepReport:
    tokens: List[tuple] = field(default_factory=list)        # (request, token) drawn in this step
    finished: List[Generation] = field(default_factory=list)
    preempted: List[int] = field(default_factory=list)
    num_tokens: int = 0                                       # tokens the step ran
    num_entries: int = 0


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
        # A step launched ahead may be dropped and run again; keys and values are then written
        # twice with the same numbers, but a state of fixed size that a mixer updates in place
        # would move twice.  Models with such state decode step by step.
        self.lookahead = bool(lookahead) and not self.pools.states
        self._ahead: Optional[_Ahead] = None
        self.steps_ahead = 0          # steps launched before their plan existed ...
        self.steps_ahead_dropped = 0  # ... and those of them whose plan turned out otherwise

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
        self.scheduler.add(int(request_id), prompt, params.to_native(self.default_eos))
        return int(request_id)

    def cancel(self, request_id: int) -> None:
        self.scheduler.cancel(int(request_id))

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> StepReport:
        plan = self.scheduler.schedule()
        report = StepReport(preempted=list(plan.preempted), num_tokens=int(plan.num_tokens),
                            num_entries=int(plan.num_entries))
        ahead, self._ahead = self._ahead, None
        if plan.empty:
            outcome = self.scheduler.complete(plan, [])
        else:
            try:
                drawn = logits = None
                if ahead is not None and ahead.serves(plan):
                    # this step was launched while the one before still ran
                    drawn, logits = ahead.drawn, ahead.logits
                    ahead = None
                else:
                    step = StepInput(requests=plan.requests, tokens=plan.tokens, counts=plan.counts, pos0=plan.starts,
                                     fresh=plan.fresh, logit_rows=plan.row_token_index)
                    logits = self.runner.run(step)
                    if logits is not None:
                        drawn = self.sampler.launch(logits, plan)
                if drawn is not None:
                    if self.lookahead:
                        self._ahead = self._launch_ahead(plan)
                    # also reads the kernels' status word
                    sampled = self.sampler.collect(drawn, logits, plan, logits_intact=self._ahead is None)
                else:
                    sampled = []
                    torch.cuda.current_stream().synchronize()
                    ops.check_kernel_status(self.model.device)
                outcome = self.scheduler.complete(plan, sampled)
                if self._ahead is not None and outcome["finished"]:
                    # a request ended on the token just read: the step launched ahead is not the next one
                    self._ahead = None
                    self.steps_ahead_dropped += 1
            except InternalError:
                self._ahead = None
                outcome = self.scheduler.fail(plan)
                self.failed += len(outcome["finished"])
                self._collect(report, outcome)
                raise
        if ahead is not None:
            self.steps_ahead_dropped += 1
        self._collect(report, outcome)
        return report

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
        requests = plan.requests
        positions = plan.starts + 1
        count = len(requests)
        logits = self.runner.run_ahead(requests, positions, self.sampler.device_tokens(count))
        if logits is None:
            return None
        self.steps_ahead += 1
        rows = None if plan.all_greedy else _RowsAhead(plan, self.scheduler.peek_uniforms(plan))
        return _Ahead(requests, positions, logits, self.sampler.launch(logits, rows), rows)

    def _collect(self, report: StepReport, outcome: dict) -> None:
        report.tokens.extend((int(r), int(t)) for r, t in outcome["tokens"])
        for item in outcome["finished"]:
            report.finished.append(Generation(
                request=int(item["request"]), tokens=[int(t) for t in item["tokens"]], finish=item["reason"],
                prompt_tokens=int(item["prompt_tokens"]), processed_tokens=int(item["processed_tokens"]),
                preemptions=int(item["preemptions"]), reused_tokens=int(item["reused_tokens"])))
            self.generations += 1

    def generate(self, prompts: Sequence[Sequence[int]], params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token=None) -> List[Generation]:
        """Run prompts (lists of token ids) to their ends; results in the order given."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise InvalidArgumentError("one SamplingParams is needed for each prompt, or one for all")
        ids = [self.add_request(prompt, p) for prompt, p in zip(prompts, params)]
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
        return {
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
