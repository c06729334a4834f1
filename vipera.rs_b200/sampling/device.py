"""Sampling on the device from the logits of a step, row by row as the scheduler's plan
says: penalties, then greedy or temperature with top-k, top-p and min-p.  Only the drawn
token ids (and a status per row) come back to the host."""
from __future__ import annotations

from typing import List

import numpy as np
import torch

from ..build import runtime_module
from ..errors import InternalError
from ..kernels import ops


class _Drawn:
    """Tokens on their way to the host: which pinned buffer, how many rows, and the event
    recorded behind the copy."""

    __slots__ = ("buffer", "rows", "event")

    def __init__(self, buffer, rows, event):
        self.buffer, self.rows, self.event = buffer, rows, event


class DeviceSampler:
    def __init__(self, device):
        self.device = device
        # two pinned buffers: a step's tokens may be read while the step after already copies its own
        size = ops._WORDS_HEAD + 2 * ops.SAMPLER_MAX_ROWS
        self._hosts = [torch.empty(size, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event() for _ in range(2)]
        self._turn = 0

    def device_tokens(self, rows: int) -> torch.Tensor:
        """Where the tokens of a launch() with `rows` rows lie on the device."""
        return ops.sampler_words(self.device, rows)[1]

    def launch(self, logits: torch.Tensor, plan) -> _Drawn:
        """Queue the draw of every row and the copy of the results; nothing waits."""
        rows = logits.shape[0]
        if rows > ops.SAMPLER_MAX_ROWS:
            raise InternalError(f"{rows} rows to sample exceed the sampler's {ops.SAMPLER_MAX_ROWS}")
        if plan is not None and plan.any_penalty:
            self._penalties(logits, plan)
        # token ids and row states land beside the kernels' status word: one copy brings all
        whole, tokens, status = ops.sampler_words(self.device, rows)
        if plan is None or plan.all_greedy:   # no plan: a greedy step launched ahead of its plan
            ops.argmax(logits, tokens, status)
        else:
            dev = self.device
            ops.sample(logits,
                       temperature=torch.from_numpy(plan.row_temperature).to(dev, non_blocking=True),
                       top_k=torch.from_numpy(plan.row_top_k).to(dev, non_blocking=True),
                       top_p=torch.from_numpy(plan.row_top_p).to(dev, non_blocking=True),
                       min_p=torch.from_numpy(plan.row_min_p).to(dev, non_blocking=True),
                       uniform=torch.from_numpy(plan.row_uniform).to(dev, non_blocking=True),
                       tokens=tokens, status=status)
        turn = self._turn
        self._turn ^= 1
        host = self._hosts[turn][:whole.numel()]
        host.copy_(whole, non_blocking=True)
        self._events[turn].record()
        return _Drawn(turn, rows, self._events[turn])

    def collect(self, drawn: _Drawn, logits: torch.Tensor, plan, logits_intact: bool = True) -> List[int]:
        """Wait for a launch()'s copy and return its tokens (rows the device could not draw
        are drawn on the host, from `logits`; ``logits_intact=False`` says that a later step
        has overwritten them, which is only allowed where no row can need them)."""
        rows = drawn.rows
        drawn.event.synchronize()
        values = self._hosts[drawn.buffer][:ops._WORDS_HEAD + 2 * rows].tolist()
        ops.raise_on_kernel_status(self.device, values[0])
        tokens = values[ops._WORDS_HEAD:ops._WORDS_HEAD + rows]
        codes = values[ops._WORDS_HEAD + rows:]
        for row, code in enumerate(codes):
            if code == ops.SAMPLE_OK:
                continue
            if code == ops.SAMPLE_NEEDS_HOST:
                if not logits_intact:
                    raise InternalError("a row needs the host sampler, but the step after has overwritten its logits")
                tokens[row] = self._host_draw(logits[row], plan, row)
            elif code == ops.SAMPLE_NO_FINITE:
                raise InternalError("no finite logits to sample from")
            else:
                raise InternalError("the distribution has no mass")
        return tokens

    def draw(self, logits: torch.Tensor, plan) -> List[int]:
        return self.collect(self.launch(logits, plan), logits, plan)

    def _host_draw(self, row_logits: torch.Tensor, plan, row: int) -> int:
        # Penalties were already applied to the row on the device.
        config = {"temperature": float(plan.row_temperature[row]), "top_k": int(plan.row_top_k[row]),
                  "top_p": float(plan.row_top_p[row]), "min_p": float(plan.row_min_p[row])}
        return int(runtime_module().draw_temperature(row_logits.cpu().numpy(), config, [],
                                                     float(plan.row_uniform[row])))

    def _penalties(self, logits: torch.Tensor, plan) -> None:
        rows = logits.shape[0]
        entry_row, entry_id, entry_count, entry_bias = [], [], [], []
        repetition = np.ones(rows, dtype=np.float32)
        presence = np.zeros(rows, dtype=np.float32)
        frequency = np.zeros(rows, dtype=np.float32)
        for row in range(rows):
            ids, counts, rep, pres, freq, bias = plan.row_penalty(row)
            repetition[row], presence[row], frequency[row] = rep, pres, freq
            merged = {int(i): [int(c), 0.0] for i, c in zip(ids, counts)}
            for token, value in bias:
                merged.setdefault(int(token), [0, 0.0])[1] = float(value)
            for token, (count, value) in merged.items():
                entry_row.append(row)
                entry_id.append(token)
                entry_count.append(count)
                entry_bias.append(value)
        if not entry_row:
            return
        dev = self.device
        ops.apply_penalties(
            logits,
            entry_row=torch.tensor(entry_row, dtype=torch.int32, device=dev),
            entry_id=torch.tensor(entry_id, dtype=torch.int32, device=dev),
            entry_count=torch.tensor(entry_count, dtype=torch.int32, device=dev),
            entry_bias=torch.tensor(entry_bias, dtype=torch.float32, device=dev),
            repetition=torch.from_numpy(repetition).to(dev), presence=torch.from_numpy(presence).to(dev),
            frequency=torch.from_numpy(frequency).to(dev))
