"""Pins oracle/vit_oracle.py (the numpy restatement) to the reference.

Two anchors:
* fixtures written by the reference's own compiled C code
  (tests/golden/*.npz, made by tests/golden/make_golden.py);
* the closed-form known answers the reference's tests/test_vision.c uses
  (label-smoothed cross-entropy :796-829, GEMM :631-659, AdamW :616-624).
"""
import glob
import os

import numpy as np
import pytest

from conftest import GOLDEN
from oracle import vit_oracle as vo

FIXTURES = sorted(path for path in glob.glob(os.path.join(GOLDEN, "*.npz"))
                  if os.path.basename(path) != "augmentation.npz")


def load(path):
    data = np.load(path)
    config = tuple(int(v) for v in data["config"])
    names = vo.parameter_names(config[6])
    pick = lambda tag: {n: data[tag + n] for n in names}
    weights = None
    if int(data["weighted"]):
        weights = (0.5 + 0.1 * np.arange(config[7])).astype(np.float32)
    return data, config, names, pick, weights


def drop_key_bias(name, array, d_model):
    """The key bias has a mathematically zero gradient (softmax is invariant to
    a shift shared by all keys), so what the float arithmetic leaves there is
    rounding noise, and Adam turns noise of any size into steps of size lr.
    Those d_model entries are therefore excluded from post-step comparisons."""
    if name.endswith("query_key_value_bias"):
        keep = np.ones(array.shape[1], bool)
        keep[d_model:2 * d_model] = False
        return array[:, keep]
    return array


def max_relative(actual, expected):
    scale = max(float(np.abs(expected).max()), 1e-6)
    return float(np.abs(actual - expected).max()) / scale


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_initialisation_matches_reference(path):
    data, config, names, pick, _ = load(path)
    ours = vo.init_parameters(config, seed=42)
    for name in names:
        # Xavier draws are bit-exact; Box-Muller goes through logf/cosf,
        # where libm and numpy may differ in the last bit.
        np.testing.assert_allclose(ours[name], data["init/" + name],
                                   rtol=0, atol=1e-8, err_msg=name)


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_loss_logits_and_gradients_match_reference(path):
    data, config, names, pick, weights = load(path)
    loss, grads, logits = vo.loss_and_gradients(
        pick("init/"), config, data["images"], data["labels"], weights,
        float(data["label_smoothing"]))
    assert abs(float(loss) - float(data["loss"])) <= 2e-6
    np.testing.assert_allclose(logits, data["logits"], rtol=0, atol=2e-6)
    for name in names:
        assert max_relative(grads[name], data["grad/" + name]) <= 2e-5, name


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_training_steps_match_reference(path):
    data, config, names, pick, weights = load(path)
    trainer = vo.Trainer(pick("init/"), config)
    losses = [trainer.train_batch(data["images"], data["labels"], 1e-3, 0.05,
                                  weights, float(data["label_smoothing"]))
              for _ in range(int(data["steps"]))]
    np.testing.assert_allclose(losses, data["step_losses"], rtol=0, atol=5e-6)
    for name in names:
        # After a few Adam steps an element moves by ~lr per step; agreement
        # well below that shows the same update rule.
        d = config[4]
        np.testing.assert_allclose(drop_key_bias(name, trainer.params[name], d),
                                   drop_key_bias(name, data["after/" + name], d),
                                   rtol=0, atol=2e-5, err_msg=name)
        assert max_relative(drop_key_bias(name, trainer.m[name], d),
                            drop_key_bias(name, data["m/" + name], d)) <= 1e-3, name
        assert max_relative(drop_key_bias(name, trainer.v[name], d),
                            drop_key_bias(name, data["v/" + name], d)) <= 1e-3, name


def test_label_smoothed_cross_entropy_closed_form():
    """Same construction as the reference's tests/test_vision.c:796-829."""
    logits = np.array([[1.0, 2.0, 0.5], [0.1, -0.3, 0.7]], np.float32)
    labels = np.array([1, 2])
    smoothing = 0.2
    loss, grad = vo.softmax_cross_entropy(logits, labels, None, smoothing)
    expected = 0.0
    for row, label in zip(logits.astype(np.float64), labels):
        log_p = row - np.log(np.exp(row).sum())
        target = np.full(3, smoothing / 3)
        target[label] += 1 - smoothing
        expected -= (target * log_p).sum()
    expected /= 2
    assert abs(float(loss) - expected) <= 1e-5
    assert abs(float(grad.sum())) <= 1e-6  # rows of p - t sum to zero


def test_gemm_known_answers():
    """tests/test_vision.c:631-659 style: small integer matrices."""
    x = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    w = np.array([[1, 0], [0, 1], [1, 1]], np.float32)
    np.testing.assert_array_equal(vo.gemm(x, w), [[4, 5], [10, 11]])
    dx, dw = vo.gemm_backward(x, w, np.ones((2, 2), np.float32))
    np.testing.assert_array_equal(dx, [[1, 1, 2], [1, 1, 2]])
    np.testing.assert_array_equal(dw, [[5, 5], [7, 7], [9, 9]])


def test_adamw_first_step_is_lr_sized():
    """tests/test_vision.c:616-624: after one step from zero moments the
    update is lr * (sign(g) + wd * w) up to epsilon."""
    w = np.array([[1.0, -2.0]], np.float32)
    g = np.array([[0.5, -0.25]], np.float32)
    w2, m, v = vo.adamw_update(w, g, np.zeros_like(w), np.zeros_like(w), 1,
                               lr=0.1, wd=0.01)
    np.testing.assert_allclose(w2, w - 0.1 * (np.sign(g) + 0.01 * w), atol=1e-6)


def test_patch_extraction_round_trip():
    rng = np.random.RandomState(0)
    images = rng.randn(3, 2 * 8 * 8).astype(np.float32)
    patches = vo.extract_patches(images, 2, 8, 8, 4)
    assert patches.shape == (3 * 4, 2 * 16)
    # element (row, c*P*P + y*P + x) is pixel (c, py*P + y, px*P + x)
    img = images.reshape(3, 2, 8, 8)
    assert patches[1 * 4 + 3, 1 * 16 + 2 * 4 + 1] == img[1, 1, 4 + 2, 4 + 1]
    back = vo.extract_patches_backward(patches, 3, 2, 8, 8, 4)
    np.testing.assert_array_equal(back, images)
