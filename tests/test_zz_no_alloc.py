"""The greedy argmax that brings its own scratch (csrc/kernels/no_alloc.h), called the way a
program that cannot allocate device memory would call it: through the exported C symbol,
with nothing but pointers.  Such a caller (a loop that must not synchronise the device, a
host that has given all device memory to its own pool) still owns its inputs and outputs;
only the scratch comes from inside the library.

Held to the library's ordinary argmax on the same logits and, independently of this library,
to torch's argmax over the finite values (ties to the lowest index), twice in a row with
different data, so that what the first call left in the shared scratch would show if it were read.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry_point():
    import vipera_rs_b200  # noqa: F401
    from vipera_rs_b200 import build

    library = ctypes.CDLL(build.kernel_library_path("sampling"))
    fn = library.vipera_argmax_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def test_static_argmax_matches_the_ordinary_one_twice():
    from vipera_rs_b200.kernels import ops

    fn = _entry_point()
    device = "cuda:0"
    stream = torch.cuda.current_stream().cuda_stream
    generator = torch.Generator(device=device).manual_seed(5)
    for call, (rows, vocab) in enumerate([(7, 50021), (64, 1003)]):
        logits = torch.randn(rows, vocab, device=device, generator=generator) * (call + 1)
        logits[0, 3] = float("nan")
        logits[1, :] = 0.5                      # a row of ties: the lowest index wins
        logits[2, vocab - 1] = logits[2, 11] = 99.0
        got = torch.full((rows,), -7, dtype=torch.int32, device=device)
        got_status = torch.full((rows,), -7, dtype=torch.int32, device=device)
        code = fn(logits.data_ptr(), rows, vocab, got.data_ptr(), got_status.data_ptr(), stream)
        assert code == 0
        want = torch.empty(rows, dtype=torch.int32, device=device)
        want_status = torch.empty(rows, dtype=torch.int32, device=device)
        ops.argmax(logits, want, want_status)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}"
        assert torch.equal(got_status, want_status), f"call {call}"
        assert int(got[1]) == 0 and int(got[2]) == 11
        # and to an argmax that shares nothing with this library: non-finite values masked out,
        # the first of equal maxima taken
        finite = torch.where(torch.isfinite(logits), logits, torch.full_like(logits, float("-inf")))
        best = finite.max(dim=1, keepdim=True).values
        index = torch.arange(vocab, device=device).expand(rows, vocab)
        first = torch.where(finite == best, index, torch.full_like(index, vocab)).min(dim=1).values
        assert torch.equal(got.long(), first), f"call {call}"
        assert int(got_status.abs().sum()) == 0
    # the optional status pointer may be null
    code = fn(logits.data_ptr(), rows, vocab, got.data_ptr(), None, stream)
    torch.cuda.synchronize()
    assert code == 0 and torch.equal(got, want)


def test_static_argmax_refuses_what_its_scratch_cannot_hold():
    fn = _entry_point()
    tokens = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    logits = torch.zeros(4, 8, device="cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(logits.data_ptr(), 1025, 8, tokens.data_ptr(), None, stream) == -2   # beyond the stated maximum
    assert fn(logits.data_ptr(), 4, 0, tokens.data_ptr(), None, stream) == -2
    assert fn(None, 4, 8, tokens.data_ptr(), None, stream) == -3
    assert fn(logits.data_ptr(), 0, 8, tokens.data_ptr(), None, stream) == 0       # nothing to do
