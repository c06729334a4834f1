"""Python face of the CUDA kernels: one function per launcher, called through ctypes.

Every function takes torch tensors that already live on the GPU, checks what the kernel
cannot check for itself (device, dtype, contiguity, extents), and launches on torch's
current stream.  There is no fallback: a tensor that is not on a CUDA device, a missing
compiler or a kernel that reports an error raises.
"""
from __future__ import annotations

import ctypes
import functools
import os
from typing import Optional

import torch

from ..build import load_kernel_library
from ..errors import InternalError, InvalidArgumentError, UnsupportedError

F32, BF16 = 0, 1
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
ROPE_NONE, ROPE_NEOX, ROPE_INTERLEAVED = 0, 1, 2
SAMPLE_OK, SAMPLE_NO_FINITE, SAMPLE_NO_MASS, SAMPLE_NEEDS_HOST = 0, 1, 2, 3

_c_int, _c_float, _c_void = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_functions = {}

_STATUS_TEXT = {
    -1: "unsupported element type",
    -2: "a size this kernel does not take",
    -3: "bad argument",
    -4: "the CUDA driver gave no entry point for tensor maps",
    -5: "a bounded wait inside the kernel ran out",
}


def _function(library: str, name: str, argtypes):
    key = (library, name)
    fn = _functions.get(key)
    if fn is None:
        fn = getattr(load_kernel_library(library), name)
        fn.argtypes = argtypes
        fn.restype = _c_int
        _functions[key] = fn
    return fn


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise UnsupportedError(f"kernels take float32 and bfloat16, not {dtype}")


def _stream() -> int:
    """The raw handle of torch's current stream on the current device."""
    try:
        return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())
    except AttributeError:  # a torch without that shortcut
        return torch.cuda.current_stream().cuda_stream


def feed_tokens(src: torch.Tensor, dst: torch.Tensor, own: int) -> None:
    """dst[i] = src[i] for i < own, src[0] for the rest of dst: a step's drawn tokens as the next
    step's input, on the device."""
    fn = _function("sampling", "vipera_feed_tokens", [_c_void, _c_void, _c_int, _c_int, _c_void])
    _check(fn(_gpu(src, "src", torch.int32), _gpu(dst, "dst", torch.int32), int(own), int(dst.numel()), _stream()),
           "feed_tokens", kernels=1)


def stream_synchronize() -> None:
    """Wait for the current stream (a direct call; torch's own builds a stream object first)."""
    fn = _function("sampling", "vipera_stream_synchronize", [_c_void])
    _check(fn(_stream()), "stream_synchronize", kernels=0)


launches = 0  # kernels launched through this module (replayed graphs add what they captured)


class KernelProfile:
    """Device time of a step by class of kernel, as the reference splits a pass into its kinds
    of work (crates/vipera-backend-cpu/src/profile.rs:226-275).  While one is installed
    (``ops.profile = KernelProfile()``) every launcher records a CUDA event behind its launch;
    the time between two events goes to the class of the later one.  Steps must then be
    launched kernel by kernel (a replayed graph launches nothing through this module)."""

    CLASSES = {
        "embed": "embed", "rmsnorm": "norm", "rope_cache": "rope_kv",
        "gemm_tc": "proj", "gemm_tc_rope": "proj", "gemv_small": "proj", "gemm_simt": "proj",
        "attention": "attention", "attention_prefill": "attention", "attention_prefill_tc": "attention",
        "attention_decode": "attention",
        "argmax": "sample", "sample": "sample", "apply_penalties": "sample", "feed_tokens": "sample",
        "logprobs": "sample",
    }
    ORDER = ("proj", "attention", "norm", "rope_kv", "embed", "sample", "other")

    def __init__(self):
        self._events = []
        self._marks = []
        self._start = None
        self.totals = {}   # kind of step -> {"steps": n, "ms": total, class: ms}

    def _event(self):
        return self._events.pop() if self._events else torch.cuda.Event(enable_timing=True)

    def begin(self) -> None:
        self._marks = []
        self._start = self._event()
        self._start.record()

    def mark(self, what: str) -> None:
        if self._start is None:
            return
        event = self._event()
        event.record()
        self._marks.append((self.CLASSES.get(what, "other"), event))

    def end(self, kind: str) -> dict:
        """Wait for the step and add it to the totals of its kind; returns the running averages."""
        if self._start is None:
            return {}
        torch.cuda.current_stream().synchronize()
        split = {}
        before = self._start
        for name, event in self._marks:
            split[name] = split.get(name, 0.0) + before.elapsed_time(event)
            before = event
        total = self._start.elapsed_time(before) if self._marks else 0.0
        self._events.extend(event for _, event in self._marks)
        self._events.append(self._start)
        self._start, self._marks = None, []
        totals = self.totals.setdefault(kind, {"steps": 0, "ms": 0.0})
        totals["steps"] += 1
        totals["ms"] += total
        for name, ms in split.items():
            totals[name] = totals.get(name, 0.0) + ms
        return totals

    def line(self, kind: str) -> str:
        totals = self.totals.get(kind)
        if not totals or not totals["steps"]:
            return f"PROFILE {kind} 0"
        steps, average = totals["steps"], totals["ms"] / totals["steps"]
        parts = [f"PROFILE {kind} {steps} {average:.3f} ms:"]
        for name in self.ORDER:
            if name in totals:
                ms = totals[name] / steps
                parts.append(f"{name} {ms:.3f}ms ({100.0 * ms / average if average else 0.0:.0f}%)")
        return " ".join(parts)


profile: Optional[KernelProfile] = None


def _check(status: int, what: str, kernels: int = 1) -> None:
    global launches
    if status == 0:
        launches += kernels
        if profile is not None:
            profile.mark(what)
        return
    if status > 0:
        text = f"CUDA error {status}"
        try:
            text = f"CUDA error {status}: " + torch.cuda.cudart().cudaGetErrorString(status)  # type: ignore[attr-defined]
        except Exception:
            pass
    else:
        text = _STATUS_TEXT.get(status, f"status {status}")
    raise InternalError(f"{what}: {text}")


def _gpu(tensor: torch.Tensor, name: str, dtype=None) -> int:
    if not tensor.is_cuda:
        raise InternalError(f"{name} is not on a CUDA device; this engine has no CPU path")
    if not tensor.is_contiguous():
        raise InvalidArgumentError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise InvalidArgumentError(f"{name} must be {dtype}, got {tensor.dtype}")
    return tensor.data_ptr()


def _opt(tensor: Optional[torch.Tensor], name: str, dtype=None):
    return None if tensor is None else _gpu(tensor, name, dtype)


# ----------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = scale * table[tokens[t], :] as float32."""
    fn = _function("rowwise", "vipera_embed",
                   [_c_void, _c_int, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_void])
    count, hidden = out.shape
    if table.shape[1] != hidden or tokens.numel() != count:
        raise InvalidArgumentError("embed: shapes of table, tokens and out do not agree")
    _check(fn(_gpu(table, "table"), dtype_code(table.dtype), _gpu(tokens, "tokens", torch.int32),
              _gpu(out, "out", torch.float32), count, hidden, table.shape[0], float(scale), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = rmsnorm(x[rows[r], :]) * weight (rows defaults to all rows in order)."""
    fn = _function("rowwise", "vipera_rmsnorm",
                   [_c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_void])
    hidden = x.shape[1]
    count = out.shape[0]
    if out.shape[1] != hidden or weight.numel() != hidden:
        raise InvalidArgumentError("rmsnorm: widths of x, weight and out do not agree")
    if rows is None and x.shape[0] != count:
        raise InvalidArgumentError("rmsnorm: x and out have different row counts")
    if rows is not None and rows.numel() != count:
        raise InvalidArgumentError("rmsnorm: one row index is needed for each output row")
    _check(fn(_gpu(x, "x", torch.float32), _gpu(weight, "weight", torch.float32),
              _opt(rows, "rows", torch.int32), _gpu(out, "out"), dtype_code(out.dtype), count, hidden,
              float(eps), _stream()), "rmsnorm")


_sm_counts = {}


def sm_count(device) -> int:
    """The number of multiprocessors of `device`, asked once."""
    key = str(device)
    count = _sm_counts.get(key)
    if count is None:
        count = _sm_counts[key] = int(torch.cuda.get_device_properties(device).multi_processor_count)
    return count


def rope_cache(qkv: torch.Tensor, q_out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int,
               positions: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], style: int,
               k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
               token_seq: Optional[torch.Tensor], block_table: Optional[torch.Tensor], page_size: int,
               write_cache: bool) -> None:
    """Rotate q and k of a float32 [tokens, (heads + 2 kv_heads) * d] product; write q to
    q_out [tokens, heads * d] and k, v into their cache pages."""
    fn = _function("rope_cache", "vipera_rope_cache",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int,
                    _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void])
    count = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise InvalidArgumentError("rope_cache: qkv width does not match the head counts")
    if q_out.shape[0] != count or q_out.shape[1] != num_heads * head_dim:
        raise InvalidArgumentError("rope_cache: q_out has the wrong shape")
    if style != ROPE_NONE:
        if cos is None or sin is None or cos.shape[1] != head_dim // 2:
            raise InvalidArgumentError("rope_cache: a cos/sin table of width d/2 is needed")
    if write_cache:
        if k_pool is None or v_pool is None or k_pool.dtype != q_out.dtype:
            raise InvalidArgumentError("rope_cache: cache pools must have the activation dtype")
        if k_pool.shape[1:] != (page_size, num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
            raise InvalidArgumentError("rope_cache: cache pools must be [pages, page_size, kv_heads, d]")
    width = 0 if block_table is None else block_table.shape[1]
    _check(fn(_gpu(qkv, "qkv", torch.float32), _gpu(q_out, "q_out"), dtype_code(q_out.dtype), count,
              num_heads, num_kv_heads, head_dim, _gpu(positions, "positions", torch.int32),
              _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), style,
              _opt(k_pool, "k_pool"), _opt(v_pool, "v_pool"), _opt(token_seq, "token_seq", torch.int32),
              _opt(block_table, "block_table", torch.int32), width, page_size, 1 if write_cache else 0,
              _stream()), "rope_cache")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_STORE,
              bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
              resid: Optional[torch.Tensor] = None) -> None:
    """a[M, K] times w[N, K] transposed, on the CUDA cores with float32 accumulation."""
    fn = _function("gemm_simt", "vipera_gemm_simt",
                   [_c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int,
                    _c_void, _c_void])
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise InvalidArgumentError(f"gemm: inner sizes differ ({k} and {w.shape[1]})")
    _check_gemm_outputs(m, n, epilogue, bias, out, resid)
    _check(fn(_gpu(a, "a"), dtype_code(a.dtype), _gpu(w, "w"), dtype_code(w.dtype), m, n, k, epilogue,
              _opt(bias, "bias", torch.float32), _opt(out, "out"),
              dtype_code(out.dtype) if out is not None else F32, _opt(resid, "resid", torch.float32),
              _stream()), "gemm_simt")


def _check_gemm_outputs(m, n, epilogue, bias, out, resid) -> None:
    if epilogue == EPI_STORE:
        if out is None or tuple(out.shape) != (m, n):
            raise InvalidArgumentError(f"gemm: out must be [{m}, {n}]")
        if bias is not None and bias.numel() != n:
            raise InvalidArgumentError("gemm: bias must have one value per output column")
    elif epilogue == EPI_RESIDUAL:
        if resid is None or tuple(resid.shape) != (m, n):
            raise InvalidArgumentError(f"gemm: resid must be [{m}, {n}]")
    elif epilogue == EPI_SWIGLU:
        if n % 32:
            raise UnsupportedError("gemm: SwiGLU needs an intermediate size that is a multiple of 16")
        if out is None or tuple(out.shape) != (m, n // 2):
            raise InvalidArgumentError(f"gemm: out must be [{m}, {n // 2}]")
    else:
        raise InvalidArgumentError(f"gemm: unknown epilogue {epilogue}")


def attention(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *,
              token_seq: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
              num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal grouped-query attention of every token of the step over its request's pages."""
    fn = _function("attention", "vipera_attention",
                   [_c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int,
                    _c_int, _c_int, _c_int, _c_float, _c_int, _c_void])
    count = q.shape[0]
    if head_dim % 16 or head_dim > 256:
        raise UnsupportedError(f"attention: head size {head_dim} is not a multiple of 16 up to 256")
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape or out.dtype != q.dtype:
        raise InvalidArgumentError("attention: q and out must be [tokens, heads * d] of one dtype")
    if k_pool.dtype != q.dtype or v_pool.shape != k_pool.shape:
        raise InvalidArgumentError("attention: cache pools must match q's dtype and each other")
    page_size = k_pool.shape[1]
    if k_pool.shape[2:] != (num_kv_heads, head_dim):
        raise InvalidArgumentError("attention: cache pools must be [pages, page_size, kv_heads, d]")
    _check(fn(_gpu(q, "q"), _gpu(out, "out"), dtype_code(q.dtype), _gpu(k_pool, "k_pool"), _gpu(v_pool, "v_pool"),
              _gpu(token_seq, "token_seq", torch.int32), _gpu(positions, "positions", torch.int32),
              _gpu(block_table, "block_table", torch.int32), block_table.shape[1], page_size, count,
              num_heads, num_kv_heads, head_dim, float(scale), int(window or 0), _stream()), "attention")


# ----------------------------------------------------------------------------------------
_argmax_scratch = {}


def argmax(logits: torch.Tensor, tokens: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """tokens[r] = index of the best finite logit of row r, ties to the lowest index."""
    fn = _function("sampling", "vipera_argmax", [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void])
    rows, vocab = logits.shape
    scratch = _argmax_scratch.get(str(logits.device))
    if scratch is None or scratch.numel() < 64 * rows:
        scratch = torch.empty(64 * max(rows, 256), dtype=torch.int32, device=logits.device)
        _argmax_scratch[str(logits.device)] = scratch
    _check(fn(_gpu(logits, "logits", torch.float32), rows, vocab, _gpu(tokens, "tokens", torch.int32),
              _opt(status, "status", torch.int32), scratch.data_ptr(), _stream()), "argmax", kernels=2)


def sample(logits: torch.Tensor, *, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, tokens: torch.Tensor, status: torch.Tensor) -> None:
    fn = _function("sampling", "vipera_sample",
                   [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void])
    rows, vocab = logits.shape
    _check(fn(_gpu(logits, "logits", torch.float32), rows, vocab,
              _gpu(temperature, "temperature", torch.float32), _gpu(top_k, "top_k", torch.int32),
              _gpu(top_p, "top_p", torch.float32), _gpu(min_p, "min_p", torch.float32),
              _gpu(uniform, "uniform", torch.float64), _gpu(tokens, "tokens", torch.int32),
              _gpu(status, "status", torch.int32), _stream()), "sample")


def logprobs(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, temperature: torch.Tensor, top_n: int):
    """Log-probabilities of ``tokens[i]`` in row ``rows[i]`` of ``logits`` at ``temperature[i]``
    (0: as 1), and the ``top_n`` most likely ids of each row with theirs.  Returns device tensors
    (chosen [n], top ids [n, top_n], top values [n, top_n])."""
    fn = _function("sampling", "vipera_logprobs",
                   [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void])
    count = rows.numel()
    chosen = torch.empty(count, dtype=torch.float32, device=logits.device)
    top_ids = torch.empty((count, max(top_n, 1)), dtype=torch.int32, device=logits.device)
    top_values = torch.empty((count, max(top_n, 1)), dtype=torch.float32, device=logits.device)
    _check(fn(_gpu(logits, "logits", torch.float32), logits.shape[1], count, _gpu(rows, "rows", torch.int32),
              _gpu(tokens, "tokens", torch.int32), _gpu(temperature, "temperature", torch.float32), int(top_n),
              chosen.data_ptr(), top_ids.data_ptr(), top_values.data_ptr(), _stream()), "logprobs")
    return chosen, top_ids[:, :top_n], top_values[:, :top_n]


def apply_penalties(logits: torch.Tensor, *, entry_row, entry_id, entry_count, entry_bias,
                    repetition, presence, frequency) -> None:
    fn = _function("sampling", "vipera_apply_penalties",
                   [_c_void, _c_int, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void])
    _check(fn(_gpu(logits, "logits", torch.float32), logits.shape[1], entry_row.numel(),
              _gpu(entry_row, "entry_row", torch.int32), _gpu(entry_id, "entry_id", torch.int32),
              _gpu(entry_count, "entry_count", torch.int32), _gpu(entry_bias, "entry_bias", torch.float32),
              _gpu(repetition, "repetition", torch.float32), _gpu(presence, "presence", torch.float32),
              _gpu(frequency, "frequency", torch.float32), _stream()), "apply_penalties")


# ----------------------------------------------------------------------------------------
# tensor-core products
# ----------------------------------------------------------------------------------------
_tc_state = {}
buffer_generation = 0  # goes up whenever a shared kernel buffer moves; captured graphs are then stale


SAMPLER_MAX_ROWS = 4096
SAMPLER_MAX_TOP_K = 4096  # the largest top-k the device sampler draws without the host (kMaxCandidates in sampling.cu)
_WORDS_HEAD = 8  # int32 words in front of the sampler's outputs; the first is the kernel status word


def _tc_buffers(device, scratch_bytes: int):
    """Scratch for the partial sums of split products and the status word of the kernels with
    bounded waits, per device.  The scratch grows on demand and is shared by all products,
    which run one after another on one stream.  The status word is the first word of a small
    buffer that also receives the sampler's token ids and row states, so that one copy to the
    host brings all three."""
    global buffer_generation
    state = _tc_state.setdefault(str(device), {"scratch": None, "status": None, "words": None})
    if state["status"] is None:
        state["words"] = torch.zeros(_WORDS_HEAD + 2 * SAMPLER_MAX_ROWS, dtype=torch.int32, device=device)
        state["status"] = state["words"][:1]
    if scratch_bytes and (state["scratch"] is None or state["scratch"].numel() * 4 < scratch_bytes):
        state["scratch"] = torch.empty(max(scratch_bytes // 4, 8 << 20), dtype=torch.float32, device=device)
        buffer_generation += 1
    return state


def sampler_words(device, rows: int):
    """(whole, tokens, states): int32 device views for `rows` sampled rows, laid out so that
    ``whole`` (the status word's neighbourhood, then tokens, then row states) is one
    contiguous copy."""
    words = _tc_buffers(device, 0)["words"]
    return (words[:_WORDS_HEAD + 2 * rows], words[_WORDS_HEAD:_WORDS_HEAD + rows],
            words[_WORDS_HEAD + rows:_WORDS_HEAD + 2 * rows])


def raise_on_kernel_status(device, code: int) -> None:
    """`code` is the status word as just read: non-zero means a bounded wait ran out."""
    if code:
        _tc_buffers(device, 0)["status"].zero_()
        _function("gemm_tc", "vipera_gemm_tc_reset", [_c_void])(_stream())
        raise InternalError(f"a tensor-core kernel gave up waiting (code {code}); the step's results are invalid")


_workspace_sizes = {}


def gemm_tc_workspace(m: int, n: int, k: int):
    size = _workspace_sizes.get((m, n, k))
    if size is None:
        fn = _function("gemm_tc", "vipera_gemm_tc_workspace",
                       [_c_int, _c_int, _c_int, ctypes.POINTER(ctypes.c_size_t)])
        scratch = ctypes.c_size_t(0)
        _check(fn(m, n, k, ctypes.byref(scratch)), "gemm_tc_workspace", kernels=0)
        if len(_workspace_sizes) > 65536:
            _workspace_sizes.clear()
        size = _workspace_sizes[(m, n, k)] = scratch.value
    return size


def _even_ok(n: int, epilogue: int, out) -> bool:
    return n % 4 == 0 and (epilogue == EPI_RESIDUAL or
                           (epilogue == EPI_STORE and out is not None and out.dtype == torch.float32))


_plans = {}


def gemm_tc_plan(m: int, n: int, k: int, epilogue: int = EPI_STORE, even_ok: bool = False):
    """The form the tensor-core product takes for these sizes: a dict with `swapped`, `tile`,
    `splits`, `even_shares` (equal shares of all k-blocks per block instead of whole tiles) and
    `blocks`.  `even_ok`: the ending is one that can take other blocks' partial sums (float32
    output or the residual stream, rows a multiple of 16 bytes)."""
    key = (int(m), int(n), int(k), int(epilogue), bool(even_ok), _even_shares_mode[0])
    plan = _plans.get(key)
    if plan is None:
        fn = _function("gemm_tc", "vipera_gemm_tc_plan", [_c_int] * 5 + [ctypes.POINTER(_c_int)])
        form = (_c_int * 6)()
        _check(fn(key[0], key[1], key[2], key[3], int(key[4]), form), "gemm_tc_plan", kernels=0)
        if len(_plans) > 65536:
            _plans.clear()
        plan = _plans[key] = {"swapped": bool(form[0]), "tile": form[1], "splits": form[2],
                              "even_shares": bool(form[3]), "blocks": form[4], "pairs": bool(form[5])}
    return plan


_even_shares_mode = [None]


def gemm_tc_even_shares(mode: int) -> int:
    """Sets when the product takes even shares (0 never, 1 where its estimate favours them, 2
    wherever the ending allows) and returns the mode before; -1 only asks."""
    before = _function("gemm_tc", "vipera_gemm_tc_even_shares", [_c_int])(int(mode))
    if mode >= 0:
        _even_shares_mode[0] = (_even_shares_mode[0], "even", int(mode))
        _workspace_sizes.clear()
    return before


def gemm_tc_pairs(mode: int) -> int:
    """Sets when the product runs on pairs of blocks that share tiles of 256 tokens (0 never, 1
    where its estimate favours them, 2 wherever the form allows) and returns the mode before; -1
    only asks."""
    before = _function("gemm_tc", "vipera_gemm_tc_pairs", [_c_int])(int(mode))
    if mode >= 0:
        _even_shares_mode[0] = (_even_shares_mode[0], "pairs", int(mode))   # a new key for the kept plans
        _workspace_sizes.clear()
    return before


def gemm_tc(a: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_STORE,
            bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
            resid: Optional[torch.Tensor] = None) -> None:
    """a[M, K] times w[N, K] transposed in bfloat16 on the tensor cores (tcgen05, TMA)."""
    fn = _function("gemm_tc", "vipera_gemm_tc",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void, _c_void,
                    ctypes.c_size_t, _c_void, _c_void])
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise InvalidArgumentError(f"gemm: inner sizes differ ({k} and {w.shape[1]})")
    if k % 8:
        raise UnsupportedError(f"gemm_tc: inner size {k} is not a multiple of 8")
    _check_gemm_outputs(m, n, epilogue, bias, out, resid)
    scratch_bytes = gemm_tc_workspace(m, n, k)
    state = _tc_buffers(a.device, scratch_bytes)
    scratch = state["scratch"]
    _check(fn(_gpu(a, "a", torch.bfloat16), _gpu(w, "w", torch.bfloat16), m, n, k, epilogue,
              _opt(bias, "bias", torch.float32), _opt(out, "out"),
              dtype_code(out.dtype) if out is not None else F32, _opt(resid, "resid", torch.float32),
              None if scratch is None else scratch.data_ptr(),
              0 if scratch is None else scratch.numel() * 4,
              state["status"].data_ptr(), _stream()), "gemm_tc",
           kernels=2 if scratch_bytes and gemm_tc_plan(m, n, k, epilogue, _even_ok(n, epilogue, out))["splits"] > 1 else 1)


class _GemmRope(ctypes.Structure):
    _fields_ = [
        ("positions", _c_void), ("token_entry", _c_void), ("block_table", _c_void), ("cos_table", _c_void),
        ("sin_table", _c_void), ("q_out", _c_void), ("k_pool", _c_void), ("v_pool", _c_void),
        ("table_width", _c_int), ("page_size", _c_int), ("num_heads", _c_int), ("num_kv_heads", _c_int),
        ("head_dim", _c_int), ("rope_style", _c_int), ("write_cache", _c_int),
    ]


_rope_takes = {}


def gemm_tc_rope_takes(tokens: int, n: int, k: int, head_dim: int) -> bool:
    """Whether the tensor-core product can end with rotation and cache write for these sizes."""
    key = (int(tokens), int(n), int(k), int(head_dim))
    known = _rope_takes.get(key)
    if known is None:
        fn = _function("gemm_tc", "vipera_gemm_tc_rope_takes", [_c_int] * 4)
        if len(_rope_takes) > 65536:
            _rope_takes.clear()
        known = _rope_takes[key] = bool(fn(*key))
    return known


def gemm_tc_rope(a: torch.Tensor, w: torch.Tensor, *, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                 num_heads: int, num_kv_heads: int, head_dim: int, positions: torch.Tensor,
                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], style: int, k_pool: torch.Tensor,
                 v_pool: torch.Tensor, token_entry: torch.Tensor, block_table: torch.Tensor, page_size: int,
                 write_cache: bool) -> None:
    """The q/k/v product of a step on the tensor cores with bias, rotation of q and k and the
    write of keys and values into their pages as its ending (bfloat16; from 192 tokens on in the
    product kernel itself, below that in the kernel that adds the partial sums of the cut K)."""
    size = _function("gemm_tc", "vipera_gemm_tc_rope_size", [])()
    if size != ctypes.sizeof(_GemmRope):
        raise InternalError("the q/k/v ending's structure differs from its Python mirror")
    fn = _function("gemm_tc", "vipera_gemm_tc_rope",
                   [_c_void, _c_void, _c_int, _c_int, _c_int, _c_void, ctypes.POINTER(_GemmRope), _c_void,
                    ctypes.c_size_t, _c_void, _c_void])
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or n != (num_heads + 2 * num_kv_heads) * head_dim:
        raise InvalidArgumentError("gemm_tc_rope: the matrix must be [(heads + 2 kv_heads) * d, K]")
    if tuple(q_out.shape) != (m, num_heads * head_dim):
        raise InvalidArgumentError("gemm_tc_rope: q_out must be [tokens, heads * d]")
    if style not in (ROPE_NONE, ROPE_NEOX):
        raise UnsupportedError("gemm_tc_rope: rotary styles none and neox")
    r = _GemmRope()
    r.positions = _gpu(positions, "positions", torch.int32)
    r.token_entry = _gpu(token_entry, "token_entry", torch.int32)
    r.block_table = _gpu(block_table, "block_table", torch.int32)
    r.cos_table = _opt(cos, "cos", torch.float32)
    r.sin_table = _opt(sin, "sin", torch.float32)
    r.q_out = _gpu(q_out, "q_out", torch.bfloat16)
    r.k_pool = _gpu(k_pool, "k_pool", torch.bfloat16)
    r.v_pool = _gpu(v_pool, "v_pool", torch.bfloat16)
    r.table_width, r.page_size = int(block_table.shape[1]), int(page_size)
    r.num_heads, r.num_kv_heads, r.head_dim = int(num_heads), int(num_kv_heads), int(head_dim)
    r.rope_style, r.write_cache = int(style), 1 if write_cache else 0
    # (fewer than 192 tokens: K is cut, and the kernel that adds the partial sums has the ending)
    scratch_bytes = gemm_tc_workspace(m, n, k)
    state = _tc_buffers(a.device, scratch_bytes)
    scratch = state["scratch"]
    _check(fn(_gpu(a, "a", torch.bfloat16), _gpu(w, "w", torch.bfloat16), m, n, k, _opt(bias, "bias", torch.float32),
              ctypes.byref(r), None if scratch is None else scratch.data_ptr(),
              0 if scratch is None else scratch.numel() * 4, state["status"].data_ptr(), _stream()), "gemm_tc_rope",
           kernels=2 if m < 192 else 1)


def wait_probe(device, limit: int = 4096) -> None:
    """Launch a block whose bounded wait runs out after `limit` polls (on a barrier nothing
    arrives at, with no copy in flight): the status word then holds what a product kernel
    writes when one of its waits gives up.  For testing how that is reported."""
    fn = _function("gemm_tc", "vipera_gemm_tc_wait_probe", [_c_void, _c_int, _c_void])
    _check(fn(kernel_status_word(device).data_ptr(), int(limit), _stream()), "wait_probe")


def check_kernel_status(device) -> None:
    """After a synchronisation: raise if a tensor-core kernel's bounded wait ran out."""
    state = _tc_state.get(str(device))
    if state is None or state["status"] is None:
        return
    raise_on_kernel_status(device, int(state["status"].item()))


# ----------------------------------------------------------------------------------------
# bfloat16 attention on the tensor cores
# ----------------------------------------------------------------------------------------
MMA_HEAD_DIMS = (64, 128)
TC_ATTENTION_HEAD_DIMS = (64, 128)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *,
                      entry_starts: torch.Tensor, entry_pos0: torch.Tensor, block_table: torch.Tensor,
                      num_entries: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                      window: int = 0, skip_single: bool = False) -> None:
    """Flash-style attention of a step whose entries bring any number of tokens (bfloat16,
    head sizes 64 and 128), on tcgen05 with accumulators in tensor memory
    (VIPERA_ATTENTION_TC=0 keeps it on the mma.sync kernel).
    ``skip_single`` leaves entries of one token out: attention_decode with ``entry_starts`` runs them."""
    if head_dim not in MMA_HEAD_DIMS:
        raise UnsupportedError(f"attention_prefill: head size {head_dim} (built: 64, 128)")
    count = q.shape[0]
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise InvalidArgumentError("attention_prefill: q and out must be [tokens, heads * d]")
    if k_pool.shape[2:] != (num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
        raise InvalidArgumentError("attention_prefill: cache pools must be [pages, page_size, kv_heads, d]")
    pointers = (_gpu(q, "q", torch.bfloat16), _gpu(out, "out", torch.bfloat16), _gpu(k_pool, "k_pool", torch.bfloat16),
                _gpu(v_pool, "v_pool", torch.bfloat16), _gpu(entry_starts, "entry_starts", torch.int32),
                _gpu(entry_pos0, "entry_pos0", torch.int32), _gpu(block_table, "block_table", torch.int32))
    sizes = (block_table.shape[1], k_pool.shape[1], num_entries, count, num_heads, num_kv_heads, head_dim,
             float(scale), int(window or 0))
    kinds = [_c_void] * 7 + [_c_int] * 7 + [_c_float, _c_int]
    skip = 1 if skip_single else 0
    if head_dim in TC_ATTENTION_HEAD_DIMS and os.environ.get("VIPERA_ATTENTION_TC", "1") != "0":
        fn = _function("attention_tc", "vipera_attention_prefill_tc", kinds + [_c_int, _c_int, _c_void, _c_void])
        _check(fn(*pointers, *sizes, k_pool.shape[0], skip, kernel_status_word(q.device).data_ptr(), _stream()),
               "attention_prefill_tc")
        return
    fn = _function("attention_mma", "vipera_attention_prefill", kinds + [_c_int, _c_void])
    _check(fn(*pointers, *sizes, skip, _stream()), "attention_prefill")


# The split-key kernel's blocks that an SM holds at once (its launch bounds and shared memory).
DECODE_BLOCKS_PER_SM = 3
# The cut by whole waves serves steps whose longest history is above DECODE_SHORT_HISTORY keys and
# whose histories hold at least DECODE_LONG_WORK rows of keys per layer (entries x KV heads x keys):
# launches of some 30 microseconds and more.
DECODE_SHORT_HISTORY = 4096
DECODE_LONG_WORK = 1 << 18


@functools.lru_cache(maxsize=4096)
def decode_splits(num_entries: int, num_kv_heads: int, max_keys: int, sm_count: int):
    """How a decode step's keys are cut: (keys per split, splits).  A block is an (entry, KV
    head, split) and folds its split 128 keys at a time, 32 for each of its four warps.

    Short launches: a split is 128 keys, so that every block asks for all its keys at once,
    before it waits for the kernel ahead, and the whole cache of the step is in flight together;
    only when that would make more than 64 splits, or more than sixteen blocks per SM, do splits
    grow.  Long histories of many entries: the kernel runs for tens of microseconds and what
    counts is that its blocks fill whole waves (the GPU holds three blocks an SM at once; 512 blocks take as long
    as 888, measured), so the cut is the one a small model of the launch's time likes best: per
    wave a fixed cost and a cost per 128 keys, which is the memory's when the wave is full and a
    block's own latency when it is not; the constants are fitted to launches timed at batch 1 to
    64 and 8,192 to 32,768 keys."""
    base = max(1, num_entries * num_kv_heads)
    if max_keys <= DECODE_SHORT_HISTORY or base * max_keys < DECODE_LONG_WORK:
        # For the next power of two of keys, the splits past the longest history included (their
        # blocks leave at once): measured, the step at batch 8 and 8,192 keys is 0.1 ms faster
        # with these 64 splits than with the 36 of the same size that hold keys.
        bound = 128
        while bound < max_keys:
            bound *= 2
        most = max(1, min(64, (16 * sm_count) // base))
        chunk = max(128, -(-bound // most))
        chunk = -(-chunk // 128) * 128
        return chunk, max(1, -(-bound // chunk))
    slots = DECODE_BLOCKS_PER_SM * max(1, sm_count)
    fixed, per_tile_full, per_tile_alone, combine, per_split = 2.7, 3.7, 2.75, 3.0, 0.02   # microseconds
    best = None
    seen = set()
    for wanted in range(1, 65):
        chunk = -(-(-(-max_keys // wanted)) // 128) * 128
        if chunk in seen:
            continue
        seen.add(chunk)
        splits = max(1, -(-max_keys // chunk))
        tiles = chunk / 128
        full, rest = divmod(base * splits, slots)
        time = full * (fixed + tiles * per_tile_full)
        if rest:
            time += fixed + tiles * max(per_tile_full * rest / slots, per_tile_alone)
        time += combine + per_split * splits
        if best is None or time < best[0] - 1e-9:
            best = (time, chunk, splits)
    return best[1], best[2]


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *,
                     positions: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int,
                     head_dim: int, scale: float, window: int, chunk: int, num_splits: int,
                     scratch: torch.Tensor, entry_starts: Optional[torch.Tensor] = None) -> None:
    """Split-key attention of the entries that bring one token (bfloat16, head sizes 64 and
    128); the partial results of the splits are combined by a second kernel.  Without
    ``entry_starts`` every entry brings one token (q and out are [entries, heads * d], positions
    one per entry).  With ``entry_starts`` [entries + 1] the step has portions too: q and out
    are [tokens, heads * d], ``positions`` holds each entry's first position, and entries of
    more than one token are skipped (attention_prefill with ``skip_single`` runs them)."""
    fn = _function("attention_mma", "vipera_attention_decode",
                   [_c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int,
                    _c_int, _c_float, _c_int, _c_int, _c_int, _c_void, ctypes.c_size_t, _c_void, _c_void])
    if head_dim not in MMA_HEAD_DIMS:
        raise UnsupportedError(f"attention_decode: head size {head_dim} (built: 64, 128)")
    count = block_table.shape[0]
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise InvalidArgumentError("attention_decode: q and out must be [rows, heads * d]")
    if k_pool.shape[2:] != (num_kv_heads, head_dim) or v_pool.shape != k_pool.shape:
        raise InvalidArgumentError("attention_decode: cache pools must be [pages, page_size, kv_heads, d]")
    if positions.numel() != count or (entry_starts is None and q.shape[0] != count):
        raise InvalidArgumentError("attention_decode: one position and one block table row per entry")
    if entry_starts is not None and entry_starts.numel() != count + 1:
        raise InvalidArgumentError("attention_decode: entry_starts must hold one more item than there are entries")
    _check(fn(_gpu(q, "q", torch.bfloat16), _gpu(out, "out", torch.bfloat16), _gpu(k_pool, "k_pool", torch.bfloat16),
              _gpu(v_pool, "v_pool", torch.bfloat16), _gpu(positions, "positions", torch.int32),
              _gpu(block_table, "block_table", torch.int32), block_table.shape[1], k_pool.shape[1], count,
              num_heads, num_kv_heads, head_dim, float(scale), int(window or 0), int(chunk), int(num_splits),
              _gpu(scratch, "scratch", torch.float32), scratch.numel(), _opt(entry_starts, "entry_starts", torch.int32),
              _stream()), "attention_decode", kernels=2)


def attention_decode_scratch_floats(num_entries: int, num_heads: int, head_dim: int, num_splits: int) -> int:
    rows = num_entries * num_heads * num_splits
    return (2 * rows + 3) // 4 * 4 + rows * head_dim


# ----------------------------------------------------------------------------------------
# products for at most 8 tokens, with the norm in front and the ending behind fused in
# ----------------------------------------------------------------------------------------
GEMV_MAX_TOKENS = 32
GEMV_STORE, GEMV_RESIDUAL, GEMV_SWIGLU, GEMV_ROPE_CACHE = 0, 1, 2, 3


def gemv_small_takes(tokens: int, k: int, n: int) -> bool:
    """Whether the small-token kernel takes `tokens` tokens against a matrix of `n` rows and
    inner size `k` (the activations a block stages must fit in its shared memory)."""
    fn = getattr(load_kernel_library("gemv_small"), "vipera_gemv_small_takes")
    fn.argtypes, fn.restype = [_c_int, _c_int, _c_int], _c_int
    return bool(fn(int(tokens), int(k), int(n)))


class _GemvParams(ctypes.Structure):
    _fields_ = [
        ("weight", _c_void), ("N", _c_int), ("K", _c_int), ("T", _c_int),
        ("x32", _c_void), ("norm_weight", _c_void), ("eps", _c_float), ("rows", _c_void), ("a16", _c_void),
        ("epilogue", _c_int), ("bias", _c_void), ("out", _c_void), ("out_dtype", _c_int), ("resid", _c_void),
        ("num_heads", _c_int), ("num_kv_heads", _c_int), ("head_dim", _c_int), ("rope_style", _c_int),
        ("positions", _c_void), ("cos_table", _c_void), ("sin_table", _c_void), ("q_out", _c_void),
        ("k_pool", _c_void), ("v_pool", _c_void), ("token_entry", _c_void), ("block_table", _c_void),
        ("table_width", _c_int), ("page_size", _c_int), ("write_cache", _c_int),
    ]


_gemv_checked = False


def gemv_small(w: torch.Tensor, *, a: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None,
               norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, rows: Optional[torch.Tensor] = None,
               tokens: Optional[int] = None, epilogue: int = GEMV_STORE, bias: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None, rope: Optional[dict] = None) -> None:
    """w[N, K] (bfloat16) times at most 32 tokens.  The input is either ``a`` (bfloat16 [T, K])
    or the float32 residual stream ``x`` with an RMSNorm (``norm_weight``, ``eps``, optional
    ``rows`` choosing which rows of x are the tokens) computed on the way.  ``rope`` holds
    the arguments of the rotary/cache ending (see GQAttention)."""
    global _gemv_checked
    fn = _function("gemv_small", "vipera_gemv_small", [ctypes.POINTER(_GemvParams), _c_void])
    if not _gemv_checked:
        size = _function("gemv_small", "vipera_gemv_params_size", [])()
        if size != ctypes.sizeof(_GemvParams):
            raise InternalError(f"gemv_small: parameter block is {ctypes.sizeof(_GemvParams)} bytes here, {size} in the kernel")
        _gemv_checked = True
    n, k = w.shape
    p = _GemvParams()
    p.weight, p.N, p.K = _gpu(w, "w", torch.bfloat16), n, k
    if (a is None) == (x is None):
        raise InvalidArgumentError("gemv_small: give either a or x")
    if a is not None:
        if a.shape[1] != k:
            raise InvalidArgumentError("gemv_small: inner sizes differ")
        p.a16, p.T = _gpu(a, "a", torch.bfloat16), a.shape[0]
    else:
        if x.shape[1] != k or norm_weight is None or norm_weight.numel() != k:
            raise InvalidArgumentError("gemv_small: x and norm_weight must have the weight's inner size")
        p.x32, p.norm_weight, p.eps = _gpu(x, "x", torch.float32), _gpu(norm_weight, "norm_weight", torch.float32), float(eps)
        p.rows = _opt(rows, "rows", torch.int32)
        p.T = int(tokens if tokens is not None else (rows.numel() if rows is not None else x.shape[0]))
    t = p.T
    if not gemv_small_takes(t, k, n):
        raise UnsupportedError(f"gemv_small does not take {t} tokens against an inner size of {k}")
    p.epilogue = epilogue
    if epilogue == GEMV_ROPE_CACHE:
        r = rope
        p.bias = _opt(bias, "bias", torch.float32)
        p.num_heads, p.num_kv_heads, p.head_dim, p.rope_style = r["num_heads"], r["num_kv_heads"], r["head_dim"], r["style"]
        p.positions = _gpu(r["positions"], "positions", torch.int32)
        p.cos_table, p.sin_table = _opt(r["cos"], "cos", torch.float32), _opt(r["sin"], "sin", torch.float32)
        q_out = r["q_out"]
        if tuple(q_out.shape) != (t, r["num_heads"] * r["head_dim"]):
            raise InvalidArgumentError("gemv_small: q_out has the wrong shape")
        p.q_out = _gpu(q_out, "q_out", torch.bfloat16)
        p.write_cache = 1 if r["write_cache"] else 0
        if r["write_cache"]:
            p.k_pool, p.v_pool = _gpu(r["k_pool"], "k_pool", torch.bfloat16), _gpu(r["v_pool"], "v_pool", torch.bfloat16)
            p.token_entry = _gpu(r["token_entry"], "token_entry", torch.int32)
            p.block_table = _gpu(r["block_table"], "block_table", torch.int32)
            p.table_width, p.page_size = r["block_table"].shape[1], r["page_size"]
    else:
        _check_gemm_outputs(t, n, epilogue, bias, out, resid)
        p.bias = _opt(bias, "bias", torch.float32) if epilogue == GEMV_STORE else None
        p.out = _opt(out, "out")
        p.out_dtype = dtype_code(out.dtype) if out is not None else F32
        p.resid = _opt(resid, "resid", torch.float32)
    _check(fn(ctypes.byref(p), _stream()), "gemv_small")


def kernel_status_word(device) -> torch.Tensor:
    """The device word in which kernels with bounded waits report that one ran out."""
    return _tc_buffers(device, 0)["status"]
