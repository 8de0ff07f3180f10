"""Gradient accumulation on the device: K micro-batches of b images through the
backend (parameter gradients zeroed once, K forward/backward passes adding into
them, one optimiser call with 1/K folded into the clip scale) must train like
the reference's CPU step on all K*b images at once.  Tolerances are those of
tests/test_backend_gpu.py for FP32 products (the reference's own: step loss
1e-3, weights 2e-4 with the noise-only key bias masked)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LR, WD, SMOOTHING = 1e-3, 0.05, 0.1
CASES = [
    # config, micro-batches, batch per micro-batch
    ((1, 28, 28, 4, 32, 4, 2, 11), 3, 4),
    ((1, 28, 28, 2, 64, 2, 1, 11), 2, 2),   # 197 tokens: the long-sequence attention path
]


def keep_mask(name, array, d_model):
    keep = np.ones(array.shape[-1], bool)
    if name.endswith("query_key_value_bias"):
        keep[d_model:2 * d_model] = False
    return keep


@pytest.mark.parametrize("config,micro_batches,batch", CASES)
def test_accumulated_device_steps_match_the_cpu_full_batch(
        config, micro_batches, batch, vit_host_module, host_lib, checker_lib, backend):
    vh = vit_host_module
    total = micro_batches * batch
    steps = 3
    images, labels = vh.synthetic_batch(total, config[1], config[2], config[7], 9)

    backend.disable()
    cpu = vh.VitHost(checker_lib, config, total)
    cpu_losses = [cpu.train_step(images, labels, LR, WD, None, SMOOTHING)
                  for _ in range(steps)]

    backend.enable()
    backend.set_gemm_precision(1)
    backend.set_gradient_accumulation(micro_batches)
    gpu = vh.VitHost(host_lib, config, batch)
    launches = backend.kernel_launches()
    gpu_losses = [gpu.train_step_accumulated(images, labels, micro_batches, LR,
                                             WD, None, SMOOTHING)
                  for _ in range(steps)]
    assert backend.kernel_launches() > launches
    np.testing.assert_allclose(gpu_losses, cpu_losses, rtol=0, atol=1e-3)
    assert gpu.steps() == [steps] * gpu.count
    expected = cpu.parameters(0)
    for name, value in gpu.parameters(0).items():
        keep = keep_mask(name, value, config[4])
        np.testing.assert_allclose(value[..., keep], expected[name][..., keep],
                                   rtol=0, atol=2e-4, err_msg=name)

    # Back to plain steps on the same backend: one batch, no stale factor.
    backend.set_gradient_accumulation(1)
    plain_gpu = gpu.train_step(images[:batch], labels[:batch], LR, WD, None,
                               SMOOTHING)
    backend.disable()
    small = vh.VitHost(checker_lib, config, batch)
    small.set_parameters(expected)
    # Same weights, fresh moments: only the loss of the step is comparable.
    plain_cpu = small.train_step(images[:batch], labels[:batch], LR, WD, None,
                                 SMOOTHING)
    assert abs(plain_gpu - plain_cpu) < 1e-3
    backend.set_gemm_precision(-1)
    gpu.close()
    cpu.close()
    small.close()


def test_accumulation_count_is_validated(backend):
    with pytest.raises(ValueError):
        backend.set_gradient_accumulation(0)
    backend.set_gradient_accumulation(1)
