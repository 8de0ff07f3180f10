"""Flash attention on the tcgen05 tensor cores (attention_tc.cu), called through
the C-ABI on plain device pointers, against the float64 oracle of the host
loops it replaces (reference src/ops.c:1297-1355, 1381-1441).

Tolerance: 2e-3 of the largest reference entry, the bound every TF32
tensor-core attention kernel of this library is held to (operands rounded to
10 mantissa bits, FP32 accumulation and softmax); the saved log-sum-exp
(base 2) to 5e-3 absolute.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import PACKAGE
from oracle import vit_oracle as vo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    return ctypes.CDLL(os.path.join(PACKAGE, "libvitb200.so"))


def dev(array):
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32)).cuda()


def ptr(tensor, offset=0):
    return ctypes.c_void_p(tensor.data_ptr() + 4 * offset)


def host(tensor):
    torch.cuda.synchronize()
    return tensor.cpu().numpy()


def size(value):
    return ctypes.c_size_t(value)


def close(actual, expected, tolerance, floor=1e-6):
    scale = max(float(np.abs(expected).max()), floor)
    error = float(np.abs(actual - expected).max()) / scale
    assert error <= tolerance, error


def expected_lse(q, k, groups, seq, hd, scale):
    scores = np.einsum("gid,gjd->gij", q.reshape(groups, seq, hd),
                       k.reshape(groups, seq, hd)) * scale
    top = scores.max(-1)
    return (np.log(np.exp(scores - top[..., None]).sum(-1)) + top) / np.log(2.0)


@pytest.mark.parametrize("accumulate", [1, 0], ids=["add", "store"])
@pytest.mark.parametrize("groups,seq,hd", [
    (2, 197, 32), (3, 197, 64), (1, 1025, 64), (2, 130, 64), (1, 1, 32),
    (2, 128, 32), (3, 64, 64), (2, 300, 32), (1, 97, 64), (2, 129, 32),
    (1, 513, 32), (150, 197, 64),
])
def test_head_major_forward_and_backward(lib, groups, seq, hd, accumulate):
    rng = np.random.RandomState(groups * seq + hd + 3)
    rows = groups * seq
    q, k, v, dout = (rng.randn(rows, hd) for _ in range(4))
    dq0, dk0, dv0 = (rng.randn(rows, hd) for _ in range(3))
    scale = 1.0 / np.sqrt(hd)
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(dout)
    to = torch.empty(rows, hd, device="cuda")
    lse = torch.empty(rows, device="cuda")
    dots = torch.empty(rows, device="cuda")
    tdq, tdk, tdv = dev(dq0), dev(dk0), dev(dv0)
    assert lib.vitb200_k_attention_tc(
        ptr(tq), ptr(tk), ptr(tv), ptr(to), ptr(lse), size(groups), size(seq),
        size(hd), ctypes.c_float(scale), size(0), size(0), size(1), None) == 0
    assert lib.vitb200_k_attention_tc_backward(
        ptr(tq), ptr(tk), ptr(tv), ptr(to), ptr(tdo), ptr(lse), ptr(tdq),
        ptr(tdk), ptr(tdv), ptr(dots), size(groups), size(seq), size(hd),
        ctypes.c_float(scale), accumulate, size(0), size(0), size(0), size(1),
        None) == 0
    p, o = vo.multi_head_attention(q, k, v, groups, seq, scale)
    close(host(to), o, 2e-3)
    np.testing.assert_allclose(host(lse).reshape(groups, seq),
                               expected_lse(q, k, groups, seq, hd, scale),
                               rtol=0, atol=5e-3)
    dq, dk, dv = vo.multi_head_attention_backward(q, k, v, p, dout, groups,
                                                  seq, scale)
    base = float(accumulate)
    # A one-token group has exactly zero dQ and dK (dS = P (dP - D) with P = 1
    # and dP = D); TF32 operands leave rounding noise there, which is measured
    # against the size of the operands instead of against zero.
    floor = 1.0 if seq == 1 else 1e-6
    close(host(tdq), base * dq0 + dq, 2e-3, floor)
    close(host(tdk), base * dk0 + dk, 2e-3, floor)
    close(host(tdv), base * dv0 + dv, 2e-3)
    assert lib.vitb200_tensor_core_status() == 0


@pytest.mark.parametrize("batch,heads,seq,hd", [
    (2, 3, 197, 64), (3, 4, 197, 32), (1, 2, 260, 64),
])
def test_token_major_operands_are_read_and_written_in_place(lib, batch, heads,
                                                            seq, hd):
    """Q, K, V as the three column blocks of the [batch*seq, 3d] projection, O
    and dO as [batch*seq, d] merged matrices, the gradients as the column
    blocks of the projection's gradient: what the training step hands over."""
    rng = np.random.RandomState(batch * heads * seq + hd)
    d = heads * hd
    groups = batch * heads
    projected = rng.randn(batch * seq, 3 * d)
    merged_grad = rng.randn(batch * seq, d)
    grad0 = rng.randn(batch * seq, 3 * d)
    scale = 1.0 / np.sqrt(hd)

    def head_major(matrix, col0):
        block = matrix[:, col0:col0 + d].reshape(batch, seq, heads, hd)
        return block.transpose(0, 2, 1, 3).reshape(groups * seq, hd)

    def token_major(tensor):
        return tensor.reshape(batch, heads, seq, hd).transpose(0, 2, 1, 3) \
            .reshape(batch * seq, d)

    q, k, v = (head_major(projected, i * d) for i in range(3))
    dout = head_major(merged_grad, 0)
    tp, tg, tgrad = dev(projected), dev(merged_grad), dev(grad0)
    merged = torch.full((batch * seq, d), 7.0, device="cuda")
    lse = torch.empty(groups * seq, device="cuda")
    dots = torch.empty(groups * seq, device="cuda")
    assert lib.vitb200_k_attention_tc(
        ptr(tp), ptr(tp, d), ptr(tp, 2 * d), ptr(merged), ptr(lse),
        size(groups), size(seq), size(hd), ctypes.c_float(scale), size(3 * d),
        size(d), size(heads), None) == 0
    assert lib.vitb200_k_attention_tc_backward(
        ptr(tp), ptr(tp, d), ptr(tp, 2 * d), ptr(merged), ptr(tg), ptr(lse),
        ptr(tgrad), ptr(tgrad, d), ptr(tgrad, 2 * d), ptr(dots), size(groups),
        size(seq), size(hd), ctypes.c_float(scale), 1, size(3 * d), size(d),
        size(3 * d), size(heads), None) == 0
    p, o = vo.multi_head_attention(q, k, v, groups, seq, scale)
    close(host(merged), token_major(o), 2e-3)
    dq, dk, dv = vo.multi_head_attention_backward(q, k, v, p, dout, groups,
                                                  seq, scale)
    expected = grad0 + np.concatenate(
        [token_major(dq), token_major(dk), token_major(dv)], axis=1)
    close(host(tgrad), expected, 2e-3)
    assert lib.vitb200_tensor_core_status() == 0


def test_rows_of_either_family_feed_either_backward_pass(lib):
    """The streaming (mma.sync) and the tcgen05 kernels keep the same
    log-sum-exp convention: a forward pass of one and a backward pass of the
    other give the oracle's gradients."""
    groups, seq, hd = 2, 197, 64
    rng = np.random.RandomState(11)
    rows = groups * seq
    q, k, v, dout = (rng.randn(rows, hd) for _ in range(4))
    scale = 1.0 / np.sqrt(hd)
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(dout)
    to = torch.empty(rows, hd, device="cuda")
    lse = torch.empty(rows, device="cuda")
    dots = torch.empty(rows, device="cuda")
    tdq, tdk, tdv = (torch.zeros(rows, hd, device="cuda") for _ in range(3))
    assert lib.vitb200_k_attention_stream(
        ptr(tq), ptr(tk), ptr(tv), ptr(to), ptr(lse), size(groups), size(seq),
        size(hd), ctypes.c_float(scale), None) == 0
    assert lib.vitb200_k_attention_tc_backward(
        ptr(tq), ptr(tk), ptr(tv), ptr(to), ptr(tdo), ptr(lse), ptr(tdq),
        ptr(tdk), ptr(tdv), ptr(dots), size(groups), size(seq), size(hd),
        ctypes.c_float(scale), 0, size(0), size(0), size(0), size(1),
        None) == 0
    p, _ = vo.multi_head_attention(q, k, v, groups, seq, scale)
    dq, dk, dv = vo.multi_head_attention_backward(q, k, v, p, dout, groups,
                                                  seq, scale)
    close(host(tdq), dq, 2e-3)
    close(host(tdk), dk, 2e-3)
    close(host(tdv), dv, 2e-3)


def test_uncovered_shapes_are_declined(lib):
    dummy = torch.zeros(64, device="cuda")
    for hd in (8, 16, 48, 128):
        assert lib.vitb200_k_attention_tc(
            ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), size(1),
            size(1), size(hd), ctypes.c_float(1.0), size(0), size(0), size(1),
            None) == -1
    # A row pitch that TMA cannot describe (not a multiple of 16 bytes).
    assert lib.vitb200_k_attention_tc(
        ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), size(1),
        size(1), size(32), ctypes.c_float(1.0), size(33), size(32), size(1),
        None) == -1
