"""The allocation-free loss entry point against the ordinary one.

Some callers cannot let a device allocation happen on their hot path (a
cudaMalloc serialises the whole device, and some hosts give a plug-in no
memory budget beyond its inputs and outputs).  For them the library offers
vitb200_k_softmax_cross_entropy_static, whose per-row scratch is a fixed array
inside the library.  This file checks, through the C ABI, that it returns what
the scratch-taking entry point returns, twice in a row (the second call finds
the array still holding the first call's values), and that it refuses more
rows than the array holds.  It is collected last on purpose.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from conftest import PACKAGE

pytestmark = pytest.mark.gpu

MAX_ROWS = 65536


def _lib():
    return ctypes.CDLL(os.path.join(PACKAGE, "libvitb200.so"))


def _dev(array):
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32)).cuda()


def _ptr(tensor):
    return ctypes.c_void_p(tensor.data_ptr())


def _run(lib, static, logits, labels, weights, smoothing, grad0):
    rows, cols = logits.shape
    z, t, g = _dev(logits), _dev(labels.astype(np.float32)), _dev(grad0)
    w = _dev(weights) if weights is not None else None
    loss = torch.zeros(1, device="cuda")
    common = [_ptr(z), _ptr(t), _ptr(w) if w is not None else None,
              ctypes.c_float(smoothing), _ptr(loss), _ptr(g)]
    size = [ctypes.c_size_t(rows), ctypes.c_size_t(cols), None]
    if static:
        status = lib.vitb200_k_softmax_cross_entropy_static(*common, *size)
    else:
        scratch = torch.empty(rows, device="cuda")
        status = lib.vitb200_k_softmax_cross_entropy(*common, _ptr(scratch), *size)
    torch.cuda.synchronize()
    assert status == 0
    return loss.cpu().numpy()[0], g.cpu().numpy()


def test_static_scratch_matches_on_two_calls_in_a_row():
    lib = _lib()
    rng = np.random.RandomState(5)
    # Second call has fewer rows than the first, so stale entries of the first
    # call sit right behind the ones the second call uses.
    for rows, cols, smoothing, weighted in [(2048, 11, 0.1, True), (700, 11, 0.0, False)]:
        logits = rng.randn(rows, cols) * 3
        labels = rng.randint(0, cols, rows)
        weights = (0.5 + 0.1 * np.arange(cols)) if weighted else None
        grad0 = rng.randn(rows, cols) * 0.01
        expected_loss, expected_grad = _run(lib, False, logits, labels, weights,
                                            smoothing, grad0)
        loss, grad = _run(lib, True, logits, labels, weights, smoothing, grad0)
        assert abs(loss - expected_loss) <= 1e-6 * max(1.0, abs(expected_loss))
        scale = max(float(np.abs(expected_grad).max()), 1e-6)
        assert float(np.abs(grad - expected_grad).max()) / scale <= 1e-6


def test_static_scratch_rejects_too_many_rows():
    lib = _lib()
    dummy = torch.zeros(16, device="cuda")
    status = lib.vitb200_k_softmax_cross_entropy_static(
        _ptr(dummy), _ptr(dummy), None, ctypes.c_float(0.0), _ptr(dummy),
        _ptr(dummy), ctypes.c_size_t(MAX_ROWS + 1), ctypes.c_size_t(11), None)
    assert status == -2


def test_static_calls_leave_the_device_memory_as_it_is_up_to_the_largest_size():
    """What the entry point is for: once the library has resolved its array on
    this device (the first call does that), further calls must not change the
    amount of free device memory, including a call at the largest accepted
    size, whose result again equals the scratch-taking entry point's."""
    lib = _lib()
    rng = np.random.RandomState(9)
    rows, cols = MAX_ROWS, 11
    logits = rng.randn(rows, cols) * 2
    labels = rng.randint(0, cols, rows)
    grad0 = np.zeros((rows, cols))
    expected_loss, expected_grad = _run(lib, False, logits, labels, None, 0.1, grad0)
    # Inputs and outputs are the caller's: they exist before the measurement.
    z, t, g = _dev(logits), _dev(labels.astype(np.float32)), _dev(grad0)
    loss = torch.zeros(1, device="cuda")
    arguments = [_ptr(z), _ptr(t), None, ctypes.c_float(0.1), _ptr(loss), _ptr(g),
                 ctypes.c_size_t(rows), ctypes.c_size_t(cols), None]
    assert lib.vitb200_k_softmax_cross_entropy_static(*arguments) == 0   # warm-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        g.zero_()
        assert lib.vitb200_k_softmax_cross_entropy_static(*arguments) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert abs(loss.cpu().numpy()[0] - expected_loss) <= 1e-6 * max(1.0, abs(expected_loss))
    scale = max(float(np.abs(expected_grad).max()), 1e-6)
    assert float(np.abs(g.cpu().numpy() - expected_grad).max()) / scale <= 1e-6
