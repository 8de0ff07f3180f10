"""Kernel-level parity: each device kernel, called through the C-ABI on plain
device pointers, against the numpy restatement of the host loop it replaces
(oracle/vit_oracle.py).  torch is used only to own device memory.

Tolerances: 1e-5 relative to the largest reference entry for FP32 elementwise
and reduction kernels; GEMM tolerances depend on the operand precision and are
stated at the test.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import PACKAGE
from oracle import vit_oracle as vo

pytestmark = pytest.mark.gpu

FP32, TF32 = 1, 2


@pytest.fixture(scope="module")
def lib():
    library = ctypes.CDLL(os.path.join(PACKAGE, "libvitb200.so"))
    for name in dir(library):
        pass
    return library


def dev(array):
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32)).cuda()


def ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def host(tensor):
    torch.cuda.synchronize()
    return tensor.cpu().numpy()


def close(actual, expected, tolerance):
    scale = max(float(np.abs(expected).max()), 1e-6)
    error = float(np.abs(actual - expected).max()) / scale
    assert error <= tolerance, error


def size(value):
    return ctypes.c_size_t(value)


@pytest.mark.parametrize("m,k,n", [
    (1, 1, 1), (7, 4, 11), (1568, 16, 128), (32, 128, 11), (100, 33, 65),
    (1600, 128, 384), (257, 512, 128), (300, 130, 70),
])
def test_gemm_fp32_forward_and_backward(lib, m, k, n):
    rng = np.random.RandomState(m + k + n)
    x, w, dy = rng.randn(m, k), rng.randn(k, n), rng.randn(m, n)
    dx0, dw0 = rng.randn(m, k), rng.randn(k, n)  # backward accumulates
    tx, tw, tdy, ty = dev(x), dev(w), dev(dy), torch.empty(m, n, device="cuda")
    tdx, tdw = dev(dx0), dev(dw0)
    assert lib.vitb200_k_gemm(ptr(tx), ptr(tw), ptr(ty), size(m), size(k),
                              size(n), FP32, None) == 0
    assert lib.vitb200_k_gemm_backward(ptr(tx), ptr(tw), ptr(tdy), ptr(tdx),
                                       ptr(tdw), size(m), size(k), size(n),
                                       FP32, None) == 0
    close(host(ty), vo.gemm(x, w), 1e-5)
    dx, dw = vo.gemm_backward(x, w, dy)
    close(host(tdx), dx0 + dx, 1e-5)
    close(host(tdw), dw0 + dw, 2e-5)


@pytest.mark.parametrize("m,k,n", [
    (128, 32, 128), (128, 128, 128), (200, 96, 160), (1600, 128, 384),
    (1000, 512, 128), (4096, 128, 512), (333, 36, 44), (102400, 128, 128),
    (257, 1024, 256), (1568, 16, 128), (300, 16, 48), (100, 48, 16),
    (16, 16, 16), (50176, 16, 128), (1024, 256, 768), (300, 512, 512),
    (2048, 256, 256), (4000, 1024, 256), (777, 288, 512), (5000, 512, 2048),
    (513, 512, 1536), (256, 256, 256), (39 * 256 + 7, 384, 1536),
    # Several rounds of tiles over the persistent grid, ragged last row tile.
    (40013, 128, 384), (50017, 512, 128), (38000, 64, 256),
    # 256-wide tiles whose last column tile is half outside the matrix.
    (1024, 384, 1152), (4000, 1536, 384), (2100, 256, 640), (6000, 384, 384),
])
def test_gemm_tf32_tensor_cores(lib, m, k, n):
    """tcgen05 kind::tf32 path: operands keep 10 mantissa bits, accumulation is
    FP32.  Bound: 2e-3 of the largest reference entry (the tolerance stated for
    TF32 products), checked against float64."""
    rng = np.random.RandomState(m + k + n)
    x, w, dy = rng.randn(m, k), rng.randn(k, n), rng.randn(m, n)
    dx0, dw0 = rng.randn(m, k), rng.randn(k, n)
    tx, tw, tdy, ty = dev(x), dev(w), dev(dy), torch.empty(m, n, device="cuda")
    tdx, tdw = dev(dx0), dev(dw0)
    assert lib.vitb200_k_gemm(ptr(tx), ptr(tw), ptr(ty), size(m), size(k),
                              size(n), TF32, None) == 0
    assert lib.vitb200_k_gemm_backward(ptr(tx), ptr(tw), ptr(tdy), ptr(tdx),
                                       ptr(tdw), size(m), size(k), size(n),
                                       TF32, None) == 0
    torch.cuda.synchronize()
    assert lib.vitb200_tensor_core_status() == 0
    close(host(ty), x @ w, 2e-3)
    close(host(tdx), dx0 + dy @ w.T, 2e-3)
    close(host(tdw), dw0 + x.T @ dy, 2e-3)


@pytest.mark.parametrize("precision", [FP32, TF32], ids=["fp32", "tf32"])
@pytest.mark.parametrize("m,k,n", [(1600, 128, 384), (300, 64, 96), (1000, 512, 128),
                                   (1000, 512, 512), (2304, 384, 1536),
                                   (40013, 128, 512), (2304, 384, 1152)])
@pytest.mark.parametrize("extra", ["bias", "bias+gelu", "bias+residual", "gelu"])
def test_gemm_fused_epilogues(lib, m, k, n, extra, precision):
    """y = x w + bias with gelu(y) or residual + y produced by the same launch
    (what ops_gemm, ops_bias_add and ops_gelu / ops_residual compute in
    sequence, reference src/vit.c:493-535)."""
    rng = np.random.RandomState(m + k + n)
    x, w, bias, res = rng.randn(m, k), rng.randn(k, n) / np.sqrt(k), rng.randn(n), rng.randn(m, n)
    tx, tw, tb, tr = dev(x), dev(w), dev(bias), dev(res)
    ty, ty2 = torch.empty(m, n, device="cuda"), torch.empty(m, n, device="cuda")
    use_bias = "bias" in extra
    assert lib.vitb200_k_gemm_fused(
        ptr(tx), ptr(tw), ptr(ty), ptr(tb) if use_bias else None,
        ptr(ty2) if "gelu" in extra else None,
        ptr(tr) if "residual" in extra else None,
        ptr(ty2) if "residual" in extra else None,
        size(m), size(k), size(n), precision, None) == 0
    torch.cuda.synchronize()
    assert lib.vitb200_tensor_core_status() == 0
    tolerance = 1e-5 if precision == FP32 else 2e-3
    y = x @ w + (bias if use_bias else 0.0)
    close(host(ty), y, tolerance)
    if "gelu" in extra:
        close(host(ty2), vo.gelu(y), tolerance)
    if "residual" in extra:
        close(host(ty2), y + res, tolerance)


@pytest.mark.parametrize("m,k,n", [
    (1600, 512, 128), (300, 96, 64), (130, 48, 32), (4096, 2048, 512),
    (25600, 512, 128), (129, 132, 36), (40013, 512, 128),
])
@pytest.mark.parametrize("with_sums", [False, True], ids=["plain", "sums"])
def test_gemm_backward_through_gelu(lib, m, k, n, with_sums):
    """d(hidden) = (dY W^T) * gelu'(hidden) in one kernel, the reference's
    gemm_backward input half followed by gelu_backward (src/vit.c:552-554),
    with the per-CTA column sums the bias gradient is taken from.  TF32
    operands: 2e-3 of the largest entry; the column sums add up to m values
    each, so they get the same relative bound against their own scale."""
    rng = np.random.RandomState(m + k + n)
    w = rng.randn(k, n) / np.sqrt(n)
    dy = rng.randn(m, n)
    hidden = rng.randn(m, k) * 1.5
    tw, tdy, th = dev(w), dev(dy), dev(hidden)
    tdh = torch.full((m, k), 7.0, device="cuda")   # stored, not accumulated
    rows = 296
    tsums = torch.full((rows, k), 3.0, device="cuda") if with_sums else None
    assert lib.vitb200_k_gemm_backward_gelu(
        ptr(tw), ptr(tdy), ptr(th), ptr(tdh), ptr(tsums) if with_sums else None,
        size(m), size(k), size(n), TF32, None) == 0
    torch.cuda.synchronize()
    assert lib.vitb200_tensor_core_status() == 0
    expected = vo.gelu_backward(hidden, dy @ w.T)
    close(host(tdh), expected, 2e-3)
    if with_sums:
        sums = host(tsums).astype(np.float64).sum(axis=0)
        # Exactly the column sums of what the kernel stored (up to FP32
        # summation order), and close to the reference's.
        stored = host(tdh).astype(np.float64).sum(axis=0)
        assert np.abs(sums - stored).max() <= 1e-4 * max(np.abs(stored).max(), 1.0)
        close(sums, expected.sum(axis=0), 5e-3)


def test_gemm_backward_through_gelu_declines_fp32(lib):
    """The fused kernel exists on the tensor-core path only; an FP32 request
    is refused with nothing written."""
    t = torch.zeros(64 * 64, device="cuda")
    out = torch.full((64 * 64,), 5.0, device="cuda")
    assert lib.vitb200_k_gemm_backward_gelu(
        ptr(t), ptr(t), ptr(t), ptr(out), None, size(64), size(64), size(64),
        FP32, None) == -1
    assert float(host(out).min()) == 5.0


def test_gemm_tf32_declines_unaligned_shapes(lib):
    """Row pitches that are not multiples of 16 bytes cannot be described to
    TMA; an explicit TF32 request is refused rather than silently changed."""
    t = torch.zeros(64 * 130, device="cuda")
    assert lib.vitb200_k_gemm(ptr(t), ptr(t), ptr(t), size(64), size(33),
                              size(130), TF32, None) == -1
    assert lib.vitb200_k_gemm(ptr(t), ptr(t), ptr(t), size(64), size(8),
                              size(64), TF32, None) == -1


@pytest.mark.parametrize("rows,cols", [
    (1, 4), (5, 32), (33, 100), (100, 128), (1600, 128), (77, 256), (64, 384),
    (50, 512), (9, 1024), (3, 2048), (10, 11),
])
def test_layer_norm_forward_and_backward(lib, rows, cols):
    rng = np.random.RandomState(rows * cols)
    x = rng.randn(rows, cols) * 2 + 0.5
    gamma, beta = rng.randn(1, cols), rng.randn(1, cols)
    dy = rng.randn(rows, cols)
    dx0, dg0, db0 = rng.randn(rows, cols), rng.randn(1, cols), rng.randn(1, cols)
    tx, tg, tb, tdy = dev(x), dev(gamma), dev(beta), dev(dy)
    ty = torch.empty(rows, cols, device="cuda")
    tdx, tdg, tdb = dev(dx0), dev(dg0), dev(db0)
    eps = ctypes.c_float(1e-5)
    lib.vitb200_k_layer_norm(ptr(tx), ptr(tg), ptr(tb), eps, ptr(ty),
                             size(rows), size(cols), None)
    lib.vitb200_k_layer_norm_backward(ptr(tx), ptr(tg), eps, ptr(tdy), ptr(tdx),
                                      ptr(tdg), ptr(tdb), size(rows),
                                      size(cols), None)
    close(host(ty), vo.layer_norm(x, gamma, beta), 1e-5)
    dx, dg, db = vo.layer_norm_backward(x, gamma, dy)
    close(host(tdx), dx0 + dx, 1e-5)
    close(host(tdg), dg0 + dg, 1e-5)
    close(host(tdb), db0 + db, 1e-5)


@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096 * 50 + 2])
def test_gelu_forward_and_backward(lib, n):
    rng = np.random.RandomState(n)
    x, dy, dx0 = rng.randn(n) * 3, rng.randn(n), rng.randn(n)
    tx, tdy, tdx = dev(x), dev(dy), dev(dx0)
    ty = torch.empty(n, device="cuda")
    lib.vitb200_k_gelu(ptr(tx), ptr(ty), size(n), None)
    lib.vitb200_k_gelu_backward(ptr(tx), ptr(tdy), ptr(tdx), size(n), None)
    close(host(ty), vo.gelu(x), 1e-5)
    close(host(tdx), dx0 + vo.gelu_backward(x, dy), 1e-5)


@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 11), (1000, 384), (40000, 128), (3, 2052)])
def test_bias_add_and_column_sums(lib, rows, cols):
    rng = np.random.RandomState(rows + cols)
    x, b, acc0 = rng.randn(rows, cols), rng.randn(1, cols), rng.randn(1, cols)
    tx, tb, tacc = dev(x), dev(b), dev(acc0)
    lib.vitb200_k_column_sums(ptr(tx), ptr(tacc), size(rows), size(cols), None)
    close(host(tacc), acc0 + x.sum(axis=0, keepdims=True), 1e-5)
    lib.vitb200_k_bias_add(ptr(tx), ptr(tb), ptr(tx), size(rows), size(cols), None)  # in place
    close(host(tx), (x + b).astype(np.float32), 1e-6)


@pytest.mark.parametrize("precision", [FP32, TF32], ids=["fp32", "tf32"])
@pytest.mark.parametrize("groups,seq,hd", [
    (1, 1, 8), (3, 5, 4), (8, 50, 8), (16, 50, 16), (4, 197, 32), (2, 197, 64),
    (2, 50, 128), (1, 257, 64), (2, 33, 24), (3, 64, 16), (2, 65, 32),
    (1, 1025, 64),
])
def test_attention_forward_and_backward(lib, groups, seq, hd, precision):
    """FP32 kernels to 1e-5 / 2e-5; TF32 tensor-core kernels (operands rounded
    to 10 mantissa bits, FP32 accumulation and softmax) to 2e-3 of the largest
    reference entry."""
    if precision == TF32 and hd not in (8, 16, 32, 64, 128):
        pytest.skip("tensor-core attention covers head dims 8..128, powers of 2")
    forward_tol, backward_tol = (1e-5, 2e-5) if precision == FP32 else (2e-3, 2e-3)
    rng = np.random.RandomState(groups * seq + hd)
    rows = groups * seq
    q, k, v, dout = (rng.randn(rows, hd) for _ in range(4))
    dq0, dk0, dv0 = (rng.randn(rows, hd) for _ in range(3))
    scale = 1.0 / np.sqrt(hd)
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(dout)
    tp = torch.empty(rows, seq, device="cuda")
    to = torch.empty(rows, hd, device="cuda")
    tdq, tdk, tdv = dev(dq0), dev(dk0), dev(dv0)
    dots = torch.empty(rows, device="cuda")
    assert lib.vitb200_k_attention(ptr(tq), ptr(tk), ptr(tv), ptr(tp), ptr(to),
                                   size(groups), size(seq), size(hd),
                                   ctypes.c_float(scale), precision, None) == 0
    assert lib.vitb200_k_attention_backward(
        ptr(tq), ptr(tk), ptr(tv), ptr(tp), ptr(to), ptr(tdo), ptr(tdq),
        ptr(tdk), ptr(tdv), ptr(dots), size(groups), size(seq), size(hd),
        ctypes.c_float(scale), precision, None) == 0
    p, o = vo.multi_head_attention(q, k, v, groups, seq, scale)
    close(host(tp), p, forward_tol)
    close(host(to), o, forward_tol)
    # The backward kernels are given the device's own P and O, as in training.
    dq, dk, dv = vo.multi_head_attention_backward(
        q, k, v, host(tp).astype(np.float64), dout, groups, seq, scale)
    close(host(tdq), dq0 + dq, backward_tol)
    close(host(tdk), dk0 + dk, backward_tol)
    close(host(tdv), dv0 + dv, backward_tol)
    np.testing.assert_allclose(host(tp).sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.parametrize("precision", [FP32, TF32], ids=["fp32", "tf32"])
@pytest.mark.parametrize("groups,seq,hd", [
    (1, 1, 16), (3, 5, 16), (16, 50, 16), (5, 64, 16), (4, 17, 32),
    (3, 50, 32), (2, 64, 32), (7, 33, 16), (300, 50, 16),
])
def test_attention_without_probability_matrix(lib, groups, seq, hd, precision):
    """P = NULL: the whole-group kernels that never write P (FP32 SIMT, or
    TF32 tensor cores with every intermediate tile in registers).  Same
    tolerances as the kernels that do write it."""
    forward_tol, backward_tol = (1e-5, 2e-5) if precision == FP32 else (2e-3, 2e-3)
    rng = np.random.RandomState(groups * seq + hd + 1)
    rows = groups * seq
    q, k, v, dout = (rng.randn(rows, hd) for _ in range(4))
    dq0, dk0, dv0 = (rng.randn(rows, hd) for _ in range(3))
    scale = 1.0 / np.sqrt(hd)
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(dout)
    to = torch.empty(rows, hd, device="cuda")
    tdq, tdk, tdv = dev(dq0), dev(dk0), dev(dv0)
    assert lib.vitb200_k_attention(ptr(tq), ptr(tk), ptr(tv), None, ptr(to),
                                   size(groups), size(seq), size(hd),
                                   ctypes.c_float(scale), precision, None) == 0
    assert lib.vitb200_k_attention_backward(
        ptr(tq), ptr(tk), ptr(tv), None, ptr(to), ptr(tdo), ptr(tdq),
        ptr(tdk), ptr(tdv), None, size(groups), size(seq), size(hd),
        ctypes.c_float(scale), precision, None) == 0
    p, o = vo.multi_head_attention(q, k, v, groups, seq, scale)
    close(host(to), o, forward_tol)
    dq, dk, dv = vo.multi_head_attention_backward(q, k, v, p, dout, groups,
                                                  seq, scale)
    close(host(tdq), dq0 + dq, backward_tol)
    close(host(tdk), dk0 + dk, backward_tol)
    close(host(tdv), dv0 + dv, backward_tol)


@pytest.mark.parametrize("groups,seq,hd", [
    (2, 197, 32), (3, 197, 64), (1, 1025, 64), (2, 64, 16), (2, 65, 16),
    (4, 50, 32), (1, 1, 16), (2, 130, 64), (5, 300, 16),
])
def test_streaming_attention(lib, groups, seq, hd):
    """Flash attention with every tile in registers (TF32): forward, saved
    log-sum-exp, and the two backward kernels, against the float64 oracle."""
    rng = np.random.RandomState(groups * seq + hd + 2)
    rows = groups * seq
    q, k, v, dout = (rng.randn(rows, hd) for _ in range(4))
    dq0, dk0, dv0 = (rng.randn(rows, hd) for _ in range(3))
    scale = 1.0 / np.sqrt(hd)
    tq, tk, tv, tdo = dev(q), dev(k), dev(v), dev(dout)
    to = torch.empty(rows, hd, device="cuda")
    lse = torch.empty(rows, device="cuda")
    dots = torch.empty(rows, device="cuda")
    tdq, tdk, tdv = dev(dq0), dev(dk0), dev(dv0)
    assert lib.vitb200_k_attention_stream(
        ptr(tq), ptr(tk), ptr(tv), ptr(to), ptr(lse), size(groups), size(seq),
        size(hd), ctypes.c_float(scale), None) == 0
    assert lib.vitb200_k_attention_stream_backward(
        ptr(tq), ptr(tk), ptr(tv), ptr(to), ptr(tdo), ptr(lse), ptr(tdq),
        ptr(tdk), ptr(tdv), ptr(dots), size(groups), size(seq), size(hd),
        ctypes.c_float(scale), None) == 0
    p, o = vo.multi_head_attention(q, k, v, groups, seq, scale)
    close(host(to), o, 2e-3)
    # Row log-sum-exp of the scaled scores, in base 2.
    scores = np.einsum("gid,gjd->gij", q.reshape(groups, seq, hd),
                       k.reshape(groups, seq, hd)) * scale
    expected_lse = (np.log(np.exp(scores - scores.max(-1, keepdims=True)).sum(-1))
                    + scores.max(-1)) / np.log(2.0)
    np.testing.assert_allclose(host(lse).reshape(groups, seq), expected_lse,
                               rtol=0, atol=5e-3)
    dq, dk, dv = vo.multi_head_attention_backward(q, k, v, p, dout, groups,
                                                  seq, scale)
    close(host(tdq), dq0 + dq, 2e-3)
    close(host(tdk), dk0 + dk, 2e-3)
    close(host(tdv), dv0 + dv, 2e-3)


def test_streaming_attention_rejects_other_head_dims(lib):
    dummy = torch.zeros(1, device="cuda")
    assert lib.vitb200_k_attention_stream(
        ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), size(1),
        size(1), size(8), ctypes.c_float(1.0), None) == -1


def test_attention_without_probability_matrix_rejects_long_sequences(lib):
    dummy = torch.zeros(1, device="cuda")
    for precision, seq in ((FP32, 129), (TF32, 65)):
        assert lib.vitb200_k_attention(ptr(dummy), ptr(dummy), ptr(dummy), None,
                                       ptr(dummy), size(1), size(seq), size(16),
                                       ctypes.c_float(1.0), precision,
                                       None) == -1


def test_attention_rejects_unsupported_head_dim(lib):
    dummy = torch.zeros(1, device="cuda")
    assert lib.vitb200_k_attention(ptr(dummy), ptr(dummy), ptr(dummy),
                                   ptr(dummy), ptr(dummy), size(1), size(1),
                                   size(129), ctypes.c_float(1.0), FP32,
                                   None) == -1


@pytest.mark.parametrize("rows,cols,smoothing,weighted", [
    (1, 11, 0.0, False), (32, 11, 0.1, False), (2048, 11, 0.1, True),
    (7, 5, 0.3, True), (9, 40, 0.05, False),
])
def test_softmax_cross_entropy(lib, rows, cols, smoothing, weighted):
    rng = np.random.RandomState(rows + cols)
    logits = rng.randn(rows, cols) * 3
    labels = rng.randint(0, cols, rows)
    weights = (0.5 + 0.1 * np.arange(cols)) if weighted else None
    grad0 = rng.randn(rows, cols) * 0.01
    tz, tt, tg = dev(logits), dev(labels.astype(np.float32)), dev(grad0)
    tw = dev(weights) if weighted else None
    tl = torch.zeros(1, device="cuda")
    scratch = torch.empty(rows, device="cuda")
    lib.vitb200_k_softmax_cross_entropy(
        ptr(tz), ptr(tt), ptr(tw) if weighted else None,
        ctypes.c_float(smoothing), ptr(tl), ptr(tg), ptr(scratch), size(rows),
        size(cols), None)
    loss, grad = vo.softmax_cross_entropy(logits, labels, weights, smoothing)
    assert abs(float(host(tl)[0]) - float(loss)) <= 1e-5 * max(1.0, abs(float(loss)))
    # Existing gradient content is folded in before the division by rows
    # (reference src/ops.c:1063-1070).
    close(host(tg), grad0 / rows + grad, 1e-5)
