"""The plain implementation against numbers the reference's own code computed.

``tests/golden/reference_ops.npz`` holds inputs and outputs of the kernels in the reference's
``crates/vipera-backend-gpu/src/layer.cu`` (straight ports of its CPU functions), run once on a
GPU by ``tests/golden/make_reference_ops.py``.  Every function of ``plain_qwen2`` that has a
counterpart there must reproduce them; the whole-model comparison of the engine then rests on
``plain_qwen2`` (tests/test_replay.py)."""
import math
import os

import numpy as np
import torch

import plain_qwen2 as plain

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_ops.npz"))


def _t(name):
    return torch.from_numpy(np.asarray(GOLDEN[name]))


def _close(got, want, tolerance):
    scale = float(want.abs().max())
    worst = float((got.double() - want.double()).abs().max())
    assert worst <= tolerance * scale, f"{worst} against a scale of {scale}"


def test_rms_norm_matches_the_reference_kernel():
    for tag in ("a", "b"):
        x, w, eps = _t(f"rmsnorm_{tag}_x"), _t(f"rmsnorm_{tag}_w"), float(GOLDEN[f"rmsnorm_{tag}_eps"])
        _close(plain.rms_norm(x.double(), w.double(), eps), _t(f"rmsnorm_{tag}_out"), 2e-6)


def test_rope_matches_the_reference_kernel():
    for tag in ("a", "b", "c"):
        x = _t(f"rope_{tag}_x")
        heads, d = x.shape
        position, base = int(GOLDEN[f"rope_{tag}_position"]), float(GOLDEN[f"rope_{tag}_base"])
        sin, cos = plain.rope_angles([position], d, base)
        got = plain.rope_neox(x.double()[None], sin, cos)[0]
        _close(got, _t(f"rope_{tag}_out"), 2e-6)


def test_attention_matches_the_reference_kernels():
    for tag in ("a", "b"):
        q, k, v = _t(f"attn_{tag}_q"), _t(f"attn_{tag}_k"), _t(f"attn_{tag}_v")
        positions = k.shape[0]
        got = plain.attention(q.double()[None], k.double(), v.double(), first_position=positions - 1)[0]
        _close(got, _t(f"attn_{tag}_out"), 3e-6)         # one block per head over the whole history
        _close(got, _t(f"attn_{tag}_split_out"), 3e-6)   # chunks of 32 positions, then the combine


def test_swiglu_and_residual_match_the_reference_kernels():
    gate, up = _t("swiglu_gate"), _t("swiglu_up")
    _close(up.double() * plain.silu(gate.double()), _t("swiglu_out"), 2e-6)
    _close(_t("add_a") + _t("add_b"), _t("add_out"), 0.0)
