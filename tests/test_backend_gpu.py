"""Parity of the B200 backend against the reference's CPU path, through the
drop-in boundary: the host's own vit_model_* functions run unmodified and
reach the kernels through the op table installed by
cuda_backend_enable_device_execution.

Tolerances.  With FP32 products they are the reference's own
(tests/test_device.c:93-119, :174, :189): loss within 1e-4, every parameter
gradient within 1e-3 of the largest reference gradient of that parameter,
per-step training loss within 1e-3.  With TF32 tensor-core products (10-bit
operand mantissas, FP32 accumulation) the bound is the one stated for TF32
paths: 2e-3 relative, applied to the loss and, per parameter, to the gradient
error over the largest reference gradient.
"""
import glob
import os
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN, REPO
from oracle import vit_oracle as vo

pytestmark = pytest.mark.gpu

LR, WD = 1e-3, 0.05
CASES = {
    # name: (config, batch, label smoothing, class weights?)
    "device_test_p4": ((1, 28, 28, 4, 32, 4, 2, 11), 8, 0.1, False),
    "device_test_p2": ((1, 28, 28, 2, 32, 4, 2, 11), 2, 0.1, True),
    "device_test_hd128": ((1, 28, 28, 4, 128, 1, 1, 11), 2, 0.0, False),
    "vit_c_b4": ((1, 28, 28, 4, 128, 8, 4, 11), 4, 0.1, False),
    "batch_of_one": ((1, 28, 28, 7, 16, 2, 2, 11), 1, 0.1, True),
    "five_classes_hd8": ((1, 28, 28, 14, 8, 1, 1, 5), 3, 0.0, False),
    "cfg3_dims_b2": ((1, 28, 28, 2, 256, 8, 2, 11), 2, 0.1, False),
}


FP32, TF32 = 1, 2
# precision -> (loss abs, gradient max-relative, step-loss abs, weights abs,
#               first-moment relative, second-moment relative)
TOLERANCE = {
    FP32: (1e-4, 1e-3, 1e-3, 2e-4, 2e-3, 4e-3),
    # TF32 forced onto every product TMA can describe, including the tiny
    # ones the default policy keeps in FP32: errors compound through the
    # layers, so the per-parameter gradient bound is 5e-3 here; the default
    # policy is held to 2e-3 in test_vit_c_full_batch_against_oracle.
    TF32: (2e-3 * 2.5, 5e-3, 5e-3, 1e-3, 2e-2, 4e-2),
}


def weights_for(classes, weighted):
    return (0.5 + 0.1 * np.arange(classes)).astype(np.float32) if weighted else None


def max_relative(actual, expected):
    scale = max(float(np.abs(expected).max()), 1e-6)
    return float(np.abs(actual - expected).max()) / scale


def drop_key_bias(name, array, d_model):
    # The key bias gradient is exactly zero in exact arithmetic (softmax shift
    # invariance); its float value is rounding noise which Adam amplifies.
    if name.endswith("query_key_value_bias"):
        keep = np.ones(array.shape[1], bool)
        keep[d_model:2 * d_model] = False
        return array[:, keep]
    return array


def test_reference_acceptance_binary_passes():
    """The reference's tests/test_device.c, compiled unmodified and linked
    against this backend instead of the reference's cuda_backend.o."""
    binary = os.path.join(REPO, "oracle", "_ref", "test_device")
    assert os.path.exists(binary), "oracle/_ref/test_device was not built"
    done = subprocess.run([binary], capture_output=True, text=True, timeout=600)
    text = done.stdout + done.stderr
    assert "unavailable" not in text, text  # a skip would also exit 0
    assert done.returncode == 0, text
    assert "CUDA device execution: ok" in text


@pytest.mark.parametrize("precision", [FP32, TF32], ids=["fp32", "tf32"])
@pytest.mark.parametrize("case", sorted(CASES))
def test_gradients_and_training_match_cpu_reference(case, precision,
                                                    vit_host_module, host_lib, checker_lib,
                                                    backend):
    vh = vit_host_module
    backend.set_gemm_precision(precision)
    (loss_tol, grad_tol, step_tol, weight_tol, m_tol, v_tol) = TOLERANCE[precision]
    config, batch, smoothing, weighted = CASES[case]
    images, labels = vh.synthetic_batch(batch, config[1], config[2], config[7], 5)
    weights = weights_for(config[7], weighted)
    d_model = config[4]

    backend.disable()
    cpu = vh.VitHost(checker_lib, config, batch)
    cpu_loss = cpu.gradients(images, labels, weights, smoothing)
    cpu_grads = cpu.parameters(1)

    backend.enable()
    launches_before = backend.kernel_launches()
    declined_before = backend.declined_ops()
    gpu = vh.VitHost(host_lib, config, batch)
    gpu_loss = gpu.gradients(images, labels, weights, smoothing)
    gpu_grads = gpu.parameters(1)
    assert backend.kernel_launches() > launches_before, "no kernel was launched"
    # Every op of the step ran in its device slot: none fell back to the
    # host's own loop.
    assert backend.declined_ops() == declined_before
    assert backend.memory_counters()["device_bytes"] > 0

    assert abs(cpu_loss - gpu_loss) <= loss_tol
    for name in cpu_grads:
        assert max_relative(gpu_grads[name], cpu_grads[name]) <= grad_tol, name

    # Second yardstick: the numpy restatement in float64.
    params64 = {k: v.astype(np.float64) for k, v in cpu.parameters(0).items()}
    loss64, grads64, _ = vo.loss_and_gradients(
        params64, config, images.astype(np.float64), labels.astype(np.int64),
        None if weights is None else weights.astype(np.float64), smoothing)
    assert abs(float(loss64) - gpu_loss) <= loss_tol
    for name in cpu_grads:
        assert max_relative(gpu_grads[name], grads64[name]) <= grad_tol, name

    # Training steps: the device model trains while enabled, the CPU model
    # after disabling, as in tests/test_device.c:183-195.
    steps = 3
    initial = cpu.parameters(0)
    gpu_losses = [gpu.train_step(images, labels, LR, WD, weights, smoothing)
                  for _ in range(steps)]
    gpu_after = gpu.parameters(0)
    gpu_m, gpu_v = gpu.parameters(2), gpu.parameters(3)
    assert gpu.steps() == [steps] * gpu.count
    assert backend.declined_ops() == declined_before
    backend.disable()
    cpu_losses = [cpu.train_step(images, labels, LR, WD, weights, smoothing)
                  for _ in range(steps)]
    np.testing.assert_allclose(gpu_losses, cpu_losses, rtol=0, atol=step_tol)
    cpu_after, cpu_m, cpu_v = cpu.parameters(0), cpu.parameters(2), cpu.parameters(3)
    for name in cpu_after:
        ours = drop_key_bias(name, gpu_after[name], d_model)
        theirs = drop_key_bias(name, cpu_after[name], d_model)
        if precision == FP32:
            np.testing.assert_allclose(ours, theirs, rtol=0, atol=weight_tol,
                                       err_msg=name)
        else:
            # Adam normalises each element's step to about lr whatever the
            # gradient's size, so an element whose gradient is below the TF32
            # rounding noise can legitimately move the other way.  Bound the
            # worst element by what `steps` opposite steps can do and require
            # the update as a whole to agree.
            start = drop_key_bias(name, initial[name], d_model)
            assert np.abs(ours - theirs).max() <= 2.02 * LR * steps, name
            moved = np.linalg.norm(theirs - start)
            assert np.linalg.norm(ours - theirs) <= 0.25 * moved + 1e-7, name
        assert max_relative(drop_key_bias(name, gpu_m[name], d_model),
                            drop_key_bias(name, cpu_m[name], d_model)) <= m_tol, name
        assert max_relative(drop_key_bias(name, gpu_v[name], d_model),
                            drop_key_bias(name, cpu_v[name], d_model)) <= v_tol, name
    assert backend.tensor_core_status() == 0
    backend.set_gemm_precision(-1)
    gpu.close()
    cpu.close()


FIXTURES = sorted(path for path in glob.glob(os.path.join(GOLDEN, "*.npz"))
                  if os.path.basename(path) != "augmentation.npz")


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_matches_committed_reference_fixtures(path, vit_host_module, host_lib,
                                              backend):
    data = np.load(path)
    config = tuple(int(v) for v in data["config"])
    weights = weights_for(config[7], int(data["weighted"]))
    smoothing = float(data["label_smoothing"])
    labels = data["labels"].astype(np.uintp)
    backend.enable()
    backend.set_gemm_precision(FP32)
    declined_before = backend.declined_ops()
    gpu = vit_host_module.VitHost(host_lib, config, int(data["batch"]))
    loss = gpu.gradients(data["images"], labels, weights, smoothing)
    assert abs(loss - float(data["loss"])) <= 1e-4
    np.testing.assert_allclose(gpu.forward(data["images"]), data["logits"],
                               rtol=0, atol=1e-4)
    loss = gpu.gradients(data["images"], labels, weights, smoothing)
    for name, grad in gpu.parameters(1).items():
        assert max_relative(grad, data["grad/" + name]) <= 1e-3, name
    losses = [gpu.train_step(data["images"], labels, LR, WD, weights, smoothing)
              for _ in range(int(data["steps"]))]
    np.testing.assert_allclose(losses, data["step_losses"], rtol=0, atol=1e-3)
    for name, value in gpu.parameters(0).items():
        np.testing.assert_allclose(
            drop_key_bias(name, value, config[4]),
            drop_key_bias(name, data["after/" + name], config[4]),
            rtol=0, atol=2e-4, err_msg=name)
    assert backend.declined_ops() == declined_before
    backend.set_gemm_precision(-1)
    gpu.close()
    backend.disable()


@pytest.mark.parametrize("config,small,copies,bias_from_producer", [
    ((1, 28, 28, 4, 128, 8, 4, 11), 32, 64, 4),    # cfg 2: batch 2048
    ((1, 28, 28, 2, 256, 8, 6, 11), 4, 128, 4),    # cfg 3: batch 512, S = 197
], ids=["cfg2", "cfg3"])
def test_bench_size_batch_is_the_small_batch_replicated(config, small, copies,
                                                        bias_from_producer,
                                                        vit_host_module,
                                                        host_lib, backend):
    """The bench workloads at full size (cfg 2: M = 102 400 token rows, 16 384
    attention groups; cfg 3: 100 864 rows of 197-token sequences; every
    large-shape kernel and fusion) checked through a size-independent
    property: a batch made of copies of a small batch has the same mean loss
    and the same mean gradients as the small batch, which the float64 oracle
    can afford.  Shipped precision policy."""
    vh = vit_host_module
    images, labels = vh.synthetic_batch(small, 28, 28, 11, 4321)
    backend.enable()
    backend.set_gemm_precision(0)
    gpu = vh.VitHost(host_lib, config, small * copies)
    init = gpu.parameters(0)
    fused_before = backend.fusion_counters()
    declined_before = backend.declined_ops()
    paths_before = backend.kernel_paths()
    loss = gpu.gradients(np.tile(images, (copies, 1)), np.tile(labels, copies),
                         None, 0.1)
    grads = gpu.parameters(1)
    fused = backend.fusion_counters()
    paths = backend.kernel_paths()
    assert backend.declined_ops() == declined_before
    assert paths["tensor_core_products"] > paths_before["tensor_core_products"]
    if config[4] // config[5] >= 32:
        # 197-token sequences with 32-wide heads: the tcgen05 attention
        # kernels, forward and backward in every block.
        assert (paths["tensor_core_attention"] -
                paths_before["tensor_core_attention"] == 2 * config[6])
        assert paths["streaming_attention"] == paths_before["streaming_attention"]
    loss64, grads64, _ = vo.loss_and_gradients(
        {k: v.astype(np.float64) for k, v in init.items()}, config,
        images.astype(np.float64), labels.astype(np.int64), None, 0.1)
    assert abs(loss - float(loss64)) <= 5e-4
    for name in grads:
        ours = drop_key_bias(name, grads[name], config[4])
        theirs = drop_key_bias(name, grads64[name], config[4])
        assert max_relative(ours, theirs) <= 2e-3, name
    # At this size everything that can ride on a neighbour does: per block the
    # attention kernels absorb merge_heads and split_heads_backward, and the
    # bias gradients come from their producers' column sums (the QKV bias
    # from the attention backward kernels, whole-group or tcgen05).
    layers = config[6]
    assert fused["head_layouts"] - fused_before["head_layouts"] == 2 * layers
    assert (fused["bias_gradients"] - fused_before["bias_gradients"] ==
            bias_from_producer * layers)
    assert backend.tensor_core_status() == 0
    backend.set_gemm_precision(-1)
    gpu.close()
    backend.disable()


@pytest.mark.parametrize("precision", [FP32, 0], ids=["fp32", "default"])
def test_vit_c_full_batch_against_oracle(precision, vit_host_module, host_lib,
                                         backend):
    """ViT-C at its real batch of 32 (the reference's headline CPU case):
    loss, all gradients and the post-step weights against the float64 oracle.
    "default" is the shipped policy, which serves this size with TF32."""
    vh = vit_host_module
    config, batch = (1, 28, 28, 4, 128, 8, 4, 11), 32
    images, labels = vh.synthetic_batch(batch, 28, 28, 11, 1234)
    loss_tol, grad_tol, _, weight_tol, _, _ = TOLERANCE[FP32 if precision == FP32 else TF32]
    if precision != FP32:
        grad_tol = 2e-3  # the bound stated for TF32 products
    backend.enable()
    backend.set_gemm_precision(precision)
    declined_before = backend.declined_ops()
    gpu = vh.VitHost(host_lib, config, batch)
    init = gpu.parameters(0)
    loss = gpu.gradients(images, labels, None, 0.1)
    grads = gpu.parameters(1)
    trainer = vo.Trainer({k: v.astype(np.float64) for k, v in init.items()}, config)
    loss64, grads64, _ = vo.loss_and_gradients(
        trainer.params, config, images.astype(np.float64),
        labels.astype(np.int64), None, 0.1)
    assert abs(loss - float(loss64)) <= loss_tol
    for name in grads:
        assert max_relative(grads[name], grads64[name]) <= grad_tol, name
    gpu_loss = gpu.train_step(images, labels, LR, WD, None, 0.1)
    ref_loss = trainer.train_batch(images.astype(np.float64),
                                   labels.astype(np.int64), LR, WD, None, 0.1)
    assert abs(gpu_loss - float(ref_loss)) <= loss_tol
    for name, value in gpu.parameters(0).items():
        ours = drop_key_bias(name, value, 128)
        theirs = drop_key_bias(name, trainer.params[name], 128)
        if precision == FP32:
            np.testing.assert_allclose(ours, theirs, rtol=0, atol=weight_tol,
                                       err_msg=name)
        else:
            # One Adam step moves every element by about lr; an element whose
            # gradient sits inside the TF32 noise may step the other way.
            start = drop_key_bias(name, init[name], 128)
            assert np.abs(ours - theirs).max() <= 2.02 * LR, name
            assert (np.linalg.norm(ours - theirs) <=
                    0.25 * np.linalg.norm(theirs - start) + 1e-7), name
    assert backend.declined_ops() == declined_before
    assert backend.tensor_core_status() == 0
    backend.set_gemm_precision(-1)
    gpu.close()
    backend.disable()


LONG_SEQUENCE_CASES = {
    # name: (config, batch): two blocks of the 64 x 64-pixel model (1025
    # tokens, d 384, head dimension 64) and of the data-parallel model (197
    # tokens, d 512, head dimension 64).
    "cfg4_dims": ((1, 64, 64, 2, 384, 6, 2, 11), 2),
    "cfg5_dims": ((1, 28, 28, 2, 512, 8, 2, 11), 2),
}


@pytest.mark.parametrize("case", sorted(LONG_SEQUENCE_CASES))
def test_long_sequence_models_against_oracle(case, vit_host_module, host_lib,
                                             backend):
    """Whole models at the dimensions of the two largest configurations
    (reference tests/test_device.c:83-139 is the pattern: loss, every
    gradient, then a training step) under the shipped precision policy,
    against the float64 oracle: 2e-3 per parameter, the bound stated for TF32
    products.  These are the shapes that reach the tcgen05 attention kernels
    through the op table (token-major operands, the saved log-sum-exp rows
    keyed by tensor), the 128 x 256 product tile (K >= 256, N a multiple of
    256) and the wide LayerNorm rows; the counters prove that those kernels
    were the ones that ran and that no op fell back to the host."""
    vh = vit_host_module
    config, batch = LONG_SEQUENCE_CASES[case]
    layers, d_model = config[6], config[4]
    images, labels = vh.synthetic_batch(batch, config[1], config[2], config[7], 77)
    backend.enable()
    backend.set_gemm_precision(0)
    declined_before = backend.declined_ops()
    paths_before = backend.kernel_paths()
    gpu = vh.VitHost(host_lib, config, batch)
    init = gpu.parameters(0)
    loss = gpu.gradients(images, labels, None, 0.1)
    grads = gpu.parameters(1)
    paths = backend.kernel_paths()
    assert backend.declined_ops() == declined_before
    assert (paths["tensor_core_attention"] - paths_before["tensor_core_attention"]
            == 2 * layers)
    assert paths["streaming_attention"] == paths_before["streaming_attention"]
    assert paths["wide_tile_products"] > paths_before["wide_tile_products"]
    trainer = vo.Trainer({k: v.astype(np.float64) for k, v in init.items()}, config)
    loss64, grads64, _ = vo.loss_and_gradients(
        trainer.params, config, images.astype(np.float64),
        labels.astype(np.int64), None, 0.1)
    assert abs(loss - float(loss64)) <= 5e-4
    for name in grads:
        ours = drop_key_bias(name, grads[name], d_model)
        theirs = drop_key_bias(name, grads64[name], d_model)
        assert max_relative(ours, theirs) <= 2e-3, name
    gpu_loss = gpu.train_step(images, labels, LR, WD, None, 0.1)
    ref_loss = trainer.train_batch(images.astype(np.float64),
                                   labels.astype(np.int64), LR, WD, None, 0.1)
    assert abs(gpu_loss - float(ref_loss)) <= 5e-4
    for name, value in gpu.parameters(0).items():
        ours = drop_key_bias(name, value, d_model)
        theirs = drop_key_bias(name, trainer.params[name], d_model)
        start = drop_key_bias(name, init[name], d_model)
        assert np.abs(ours - theirs).max() <= 2.02 * LR, name
        assert (np.linalg.norm(ours - theirs) <=
                0.25 * np.linalg.norm(theirs - start) + 1e-7), name
    assert backend.declined_ops() == declined_before
    assert backend.tensor_core_status() == 0
    backend.set_gemm_precision(-1)
    gpu.close()
    backend.disable()


def test_single_parameter_optimiser_and_clipping_slots(vit_host_module, host_lib,
                                                       checker_lib, backend):
    """ops_adamw_step (reference src/ops.c:1102-1121; its own test,
    tests/test_vision.c:616-624, expects a decayed value and step == 1) and
    ops_clip_gradient_norm (src/ops.c:588-617) through their device slots,
    against the same calls on the CPU library."""
    import ctypes
    floats = ctypes.POINTER(ctypes.c_float)

    def adamw(lib, values, gradient, steps):
        rows, cols = values.shape
        out = [np.zeros_like(values) for _ in range(3)]
        step = ctypes.c_size_t()
        lib.vithost_adamw_single.restype = ctypes.c_int
        lib.vithost_adamw_single.argtypes = [floats, floats] + \
            [ctypes.c_size_t] * 3 + [ctypes.c_float] * 5 + [floats] * 3 + \
            [ctypes.POINTER(ctypes.c_size_t)]
        status = lib.vithost_adamw_single(
            values.ctypes.data_as(floats), gradient.ctypes.data_as(floats), rows,
            cols, steps, 0.01, 0.9, 0.999, 1e-8, 0.01,
            *[o.ctypes.data_as(floats) for o in out], ctypes.byref(step))
        assert status == 0
        return out, int(step.value)

    def clip(lib, gradients, max_norm):
        copies = [g.copy() for g in gradients]
        pointers = (floats * len(copies))(*[c.ctypes.data_as(floats) for c in copies])
        counts = (ctypes.c_size_t * len(copies))(*[c.size for c in copies])
        lib.vithost_clip_gradients.restype = ctypes.c_int
        lib.vithost_clip_gradients.argtypes = [
            ctypes.POINTER(floats), ctypes.POINTER(ctypes.c_size_t),
            ctypes.c_size_t, ctypes.c_float]
        assert lib.vithost_clip_gradients(pointers, counts, len(copies),
                                          max_norm) == 0
        return copies

    rng = np.random.RandomState(5)
    backend.enable()
    declined_before = backend.declined_ops()
    launches_before = backend.kernel_launches()
    # The reference's own known answer: one step on value 1, gradient 1.
    one = np.ones((1, 1), np.float32)
    (value, m, v), step = adamw(host_lib, one, one, 1)
    assert step == 1 and value[0, 0] < 1.0
    assert abs(value[0, 0] - (1.0 - 0.01 * (1.0 + 0.01 * 1.0))) <= 1e-6
    assert abs(m[0, 0] - 0.1) <= 1e-7 and abs(v[0, 0] - 0.001) <= 1e-7
    for shape, steps in (((3, 5), 1), ((257, 130), 4), ((1, 70001), 2)):
        values = rng.randn(*shape).astype(np.float32)
        gradient = rng.randn(*shape).astype(np.float32)
        ours, our_step = adamw(host_lib, values, gradient, steps)
        theirs, their_step = adamw(checker_lib, values, gradient, steps)
        assert our_step == their_step == steps
        for a, b, tolerance in zip(ours, theirs, (1e-6, 1e-6, 1e-7)):
            np.testing.assert_allclose(a, b, rtol=1e-5, atol=tolerance)
    gradients = [rng.randn(n).astype(np.float32) for n in (7, 4096, 100001)]
    for max_norm in (1.0, 1e6):   # clipped, and left alone
        ours = clip(host_lib, gradients, max_norm)
        theirs = clip(checker_lib, gradients, max_norm)
        for a, b in zip(ours, theirs):
            np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-8)
    assert backend.kernel_launches() > launches_before
    assert backend.declined_ops() == declined_before
    backend.disable()


def test_host_writes_and_reads_stay_coherent(vit_host_module, host_lib, backend):
    """After a synchronise the host may read or write any tensor byte; the
    next device op must see host writes (the reference's managed-memory
    contract, kept here with explicit device buffers)."""
    vh = vit_host_module
    config, batch = (1, 28, 28, 7, 16, 2, 1, 11), 2
    images, labels = vh.synthetic_batch(batch, 28, 28, 11, 9)
    backend.enable()
    gpu = vh.VitHost(host_lib, config, batch)
    before = backend.memory_counters()
    first = gpu.forward(images)
    # Host overwrites every weight with a scaled copy; the device must pick
    # the new values up on the next forward pass.
    scaled = {k: v * np.float32(0.5) for k, v in gpu.parameters(0).items()}
    gpu.set_parameters(scaled)
    second = gpu.forward(images)
    logits64, _ = vo.forward({k: v.astype(np.float64) for k, v in scaled.items()},
                             config, images.astype(np.float64))
    np.testing.assert_allclose(second, logits64, rtol=0, atol=1e-4)
    assert not np.allclose(first, second)
    after = backend.memory_counters()
    assert after["h2d_copies"] > before["h2d_copies"]
    assert after["faults"] > before["faults"]
    # Steady state: a training step moves only images, labels and the loss.
    gpu.train_step(images, labels, LR, WD, None, 0.1)
    a = backend.memory_counters()
    gpu.train_step(images, labels, LR, WD, None, 0.1)
    b = backend.memory_counters()
    assert b["h2d_bytes"] - a["h2d_bytes"] == images.nbytes + 4 * batch
    assert b["d2h_bytes"] - a["d2h_bytes"] == 4
    gpu.close()
    backend.disable()


def test_deferred_synchronize_changes_timing_not_results(vit_host_module, host_lib,
                                                         backend):
    """With the `synchronize` slot deferred the host runs ahead of the device
    (it refills the input tensors while the backward pass of the step before is
    still running); page protection and the prefetched loss keep every value
    the host sees equal to the run that waits in the slot, up to the order of
    the floating-point atomics inside the kernels (two runs of either kind
    differ by as much: 1e-6 relative).  A different batch every step: an upload
    that overtook, or was overtaken by, the host's next write would move the
    losses in the second decimal."""
    vh = vit_host_module
    config, batch, steps = (1, 28, 28, 4, 64, 4, 2, 11), 96, 6
    batches = [vh.synthetic_batch(batch, 28, 28, 11, 700 + i) for i in range(steps)]
    backend.enable()
    results = []
    for deferred in (0, 1):
        assert backend.set_deferred_synchronize(deferred) in (0, 1)
        gpu = vh.VitHost(host_lib, config, batch)
        before = backend.memory_counters()
        fills_before = backend.zero_fill_counters()
        losses = [gpu.train_step(images, labels, LR, WD, None, 0.1)
                  for images, labels in batches]
        moved = backend.memory_counters()
        # Nothing but the batch, the labels and the loss crosses the bus.
        assert (moved["d2h_bytes"] - before["d2h_bytes"]) == 4 * steps
        fills = backend.zero_fill_counters()
        # With the slot deferred every loss read is served by its prefetch.
        assert (fills["prefetched_reads"] - fills_before["prefetched_reads"] ==
                (steps if deferred else 0))
        # From the second step on (the buffers exist by then) the zeros every
        # accumulating kernel needs come from the batched fill: no memset
        # nodes between the kernels of a step.  All gradients of this model
        # are below the batched fill's size limit.
        assert fills["batched"] - fills_before["batched"] >= 15 * (steps - 1)
        assert fills["memsets"] - fills_before["memsets"] <= 60
        results.append((losses, gpu.parameters(0), gpu.parameters(2)))
        gpu.close()
    assert backend.set_deferred_synchronize(0) == 1
    strict, deferred = results
    np.testing.assert_allclose(deferred[0], strict[0], rtol=2e-5, atol=0)
    assert np.abs(np.diff(strict[0])).min() > 1e-3
    for which in (1, 2):
        for name in strict[which]:
            ours = drop_key_bias(name, deferred[which][name], config[4])
            theirs = drop_key_bias(name, strict[which][name], config[4])
            assert max_relative(ours, theirs) <= 5e-3, name
    assert backend.tensor_core_status() == 0
    backend.disable()


def test_tensors_allocated_before_enable_fall_back_to_cpu(vit_host_module,
                                                          host_lib, backend):
    """Ops on calloc'ed tensors are declined (non-zero return), so the host
    runs its own loops and results do not change (reference src/ops.c:61-64)."""
    vh = vit_host_module
    config, batch = (1, 28, 28, 7, 16, 2, 1, 11), 2
    images, labels = vh.synthetic_batch(batch, 28, 28, 11, 9)
    backend.disable()
    cpu = vh.VitHost(host_lib, config, batch)   # the driving library, on purpose
    expected = cpu.gradients(images, labels, None, 0.1)
    expected_grads = cpu.parameters(1)
    backend.enable()
    launches = backend.kernel_launches()
    declined = backend.declined_ops()
    again = cpu.gradients(images, labels, None, 0.1)
    assert again == expected
    assert backend.kernel_launches() == launches
    assert backend.declined_ops() > declined
    for name, grad in cpu.parameters(1).items():
        np.testing.assert_array_equal(grad, expected_grads[name])
    backend.disable()
    cpu.close()


def test_evaluation_and_prediction_match_cpu_reference(vit_host_module, host_lib, checker_lib,
                                                       backend):
    """The reference's inference entry points (vit_model_evaluate,
    vit_model_predict_probabilities: 256-sample chunks plus a remainder, cache
    allocated and freed inside the call) through the backend."""
    vh = vit_host_module
    config, samples = (1, 28, 28, 4, 32, 4, 2, 11), 300
    images, labels = vh.synthetic_batch(samples, 28, 28, 11, 17)
    backend.disable()
    cpu = vh.VitHost(checker_lib, config, 1)
    cpu_accuracy, cpu_loss, cpu_rate = cpu.evaluate(images, labels)
    cpu_probabilities = cpu.predict(images[:40])
    backend.enable()
    backend.set_gemm_precision(FP32)
    launches = backend.kernel_launches()
    gpu = vh.VitHost(host_lib, config, 1)
    gpu_accuracy, gpu_loss, gpu_rate = gpu.evaluate(images, labels)
    gpu_probabilities = gpu.predict(images[:40])
    assert backend.kernel_launches() > launches
    assert abs(gpu_loss - cpu_loss) <= 1e-4
    assert abs(gpu_accuracy - cpu_accuracy) <= 1.0 / samples
    np.testing.assert_allclose(gpu_probabilities, cpu_probabilities, rtol=0,
                               atol=1e-5)
    np.testing.assert_allclose(gpu_probabilities.sum(axis=1), 1.0, atol=1e-5)
    assert gpu_rate > 0 and cpu_rate > 0
    backend.set_gemm_precision(-1)
    gpu.close()
    cpu.close()
    backend.disable()


def test_unread_tensors_are_not_computed_but_reads_see_them(vit_host_module,
                                                            host_lib, checker_lib, backend):
    """The probability matrix of short-sequence attention is only defined, not
    written, during training; a host read still returns the right values, and
    the activation gradients that are zeroed every step are never filled."""
    vh = vit_host_module
    config, batch = (1, 28, 28, 4, 32, 4, 2, 11), 4
    images, labels = vh.synthetic_batch(batch, 28, 28, 11, 3)
    backend.disable()
    cpu = vh.VitHost(checker_lib, config, batch)
    cpu.train_step(images, labels, LR, WD, None, 0.1)
    backend.enable()
    backend.set_gemm_precision(FP32)
    gpu = vh.VitHost(host_lib, config, batch)
    before = backend.elision_counters()
    fused_before = backend.fusion_counters()
    gpu.train_step(images, labels, LR, WD, None, 0.1)
    gpu.train_step(images, labels, LR, WD, None, 0.1)
    after = backend.elision_counters()
    fused = backend.fusion_counters()
    layers = config[6]
    # Per block and step: merge_heads and split_heads_backward ride on the
    # attention kernels, and three of the four bias gradients come from sums
    # their matrix's producer made (layer_norm_backward twice, gelu_backward).
    assert fused["head_layouts"] - fused_before["head_layouts"] == 2 * 2 * layers
    assert fused["bias_gradients"] - fused_before["bias_gradients"] == 2 * 3 * layers
    # (The fourth, the QKV bias, also comes from its producer when the
    # tensor-core attention kernels run; this test pins the FP32 policy.)
    # Per block and step: P; the head-major Q, K, V and attention output
    # (views of the projected / merged matrices); and the same five gradients
    # less P's, which nobody produces.
    # On top of those, the gradients that residual_backward and
    # accumulate_gradient would merely copy (four per block) are aliases.
    per_block = 1 + 4 + 4 + 4
    assert after["lazy_defined"] - before["lazy_defined"] == 2 * per_block * layers
    assert after["lazy_materialised"] == before["lazy_materialised"]
    # Every definition of step 1 has been dropped (overwritten, re-zeroed or
    # summed into), and the two aliases per block that layer_norm_backward
    # sums into are dropped within their own step.
    assert after["lazy_dropped"] - before["lazy_dropped"] == (per_block + 2) * layers
    assert after["zero_fills_elided"] > before["zero_fills_elided"]
    # A host read of P forces the computation, for that tensor only.  The
    # second step started from the first step's weights, so compare with a CPU
    # model after the same two steps.
    cpu.train_step(images, labels, LR, WD, None, 0.1)
    for layer in range(layers):
        ours = gpu.block_tensor(layer, "probabilities")
        theirs = cpu.block_tensor(layer, "probabilities")
        np.testing.assert_allclose(ours, theirs, rtol=0, atol=2e-5)
        np.testing.assert_allclose(ours.sum(axis=1), 1.0, atol=1e-5)
    final = backend.elision_counters()
    assert final["lazy_materialised"] - after["lazy_materialised"] == layers
    # The head-major tensors that were never written read back correctly too,
    # values and gradients.
    for layer in range(layers):
        for name in ("query", "key", "value", "attended", "mlp_branch",
                     "attention_branch"):
            for grad in (False, True):
                ours = gpu.block_tensor(layer, name, grad)
                theirs = cpu.block_tensor(layer, name, grad)
                scale = float(np.abs(theirs).max())
                assert scale > 0
                np.testing.assert_allclose(ours, theirs, rtol=0,
                                           atol=2e-4 * scale + 1e-7,
                                           err_msg=f"{name} grad={grad}")
    reread = backend.elision_counters()
    # (8 head views; the two branch gradients are aliases.)
    assert reread["lazy_materialised"] - final["lazy_materialised"] == 10 * layers
    # Training continues correctly after the read.
    gpu_loss = gpu.train_step(images, labels, LR, WD, None, 0.1)
    cpu_loss = cpu.train_step(images, labels, LR, WD, None, 0.1)
    assert abs(gpu_loss - cpu_loss) <= 1e-3
    backend.set_gemm_precision(-1)
    gpu.close()
    cpu.close()
    backend.disable()


def test_gelu_backward_rides_on_the_product_before_it(vit_host_module, host_lib, checker_lib,
                                                      backend):
    """With tensor-core products, the gradient of the GELU output is never
    stored: the product that would write it applies the GELU's slope in its
    epilogue (reference src/vit.c:552-554 as one kernel).  The gradient before
    the GELU, the bias gradient taken from the kernel's column sums, a host
    read of the skipped gradient and the following steps all agree with the
    CPU path."""
    vh = vit_host_module
    config, batch = (1, 28, 28, 4, 64, 4, 2, 11), 16
    layers = config[6]
    images, labels = vh.synthetic_batch(batch, 28, 28, 11, 5)
    backend.disable()
    cpu = vh.VitHost(checker_lib, config, batch)
    backend.enable()
    backend.set_gemm_precision(TF32)
    gpu = vh.VitHost(host_lib, config, batch)
    # (The first step uploads the parameters as they are first used, which
    # launches held-back products early; the counts below are a later step's.)
    gpu.train_step(images, labels, LR, WD, None, 0.1)
    cpu.train_step(images, labels, LR, WD, None, 0.1)
    for step in range(2):
        before = backend.elision_counters()
        fused_before = backend.fusion_counters()
        gpu_loss = gpu.train_step(images, labels, LR, WD, None, 0.1)
        cpu_loss = cpu.train_step(images, labels, LR, WD, None, 0.1)
        after = backend.elision_counters()
        fused = backend.fusion_counters()
        assert abs(gpu_loss - cpu_loss) <= 5e-3
        # Forward: the bias of the patch embedding, of the classifier and of
        # each block's four products, and the GELU; backward: the GELU's slope
        # on each block's second MLP product.
        assert fused["epilogues"] - fused_before["epilogues"] == 2 + (5 + 1) * layers
        assert fused["bias_gradients"] - fused_before["bias_gradients"] == 4 * layers
        assert after["lazy_materialised"] == before["lazy_materialised"]
    for layer in range(layers):
        for name in ("hidden", "activated"):
            ours = gpu.block_tensor(layer, name, True)
            theirs = cpu.block_tensor(layer, name, True)
            scale = float(np.abs(theirs).max())
            assert scale > 0
            np.testing.assert_allclose(ours, theirs, rtol=0, atol=1e-2 * scale,
                                       err_msg=name)
    reread = backend.elision_counters()
    # Only the skipped gradient had to be computed for the read.
    assert reread["lazy_materialised"] - after["lazy_materialised"] == layers
    gpu_loss = gpu.train_step(images, labels, LR, WD, None, 0.1)
    cpu_loss = cpu.train_step(images, labels, LR, WD, None, 0.1)
    assert abs(gpu_loss - cpu_loss) <= 5e-3
    assert backend.tensor_core_status() == 0
    backend.set_gemm_precision(-1)
    gpu.close()
    cpu.close()
    backend.disable()


def test_device_memory_is_steady_over_many_steps(vit_host_module, host_lib, backend):
    """Pooled buffers, snapshots of overwritten sources and per-tensor scratch
    must reach a steady state: after a few steps, further training steps and
    evaluation calls (which create and free a whole activation cache each)
    allocate nothing more on the device."""
    import torch
    vh = vit_host_module
    config, batch = (1, 28, 28, 4, 64, 4, 2, 11), 64
    images, labels = vh.synthetic_batch(batch, 28, 28, 11, 9)
    backend.enable()
    backend.set_gemm_precision(0)
    gpu = vh.VitHost(host_lib, config, batch)
    for _ in range(4):
        gpu.train_step(images, labels, LR, WD, None, 0.1)
        gpu.evaluate(images, labels)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    counters_before = backend.memory_counters()
    for _ in range(25):
        gpu.train_step(images, labels, LR, WD, None, 0.1)
        gpu.evaluate(images, labels)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    counters_after = backend.memory_counters()
    assert free_after >= free_before - (1 << 20), (free_before, free_after)
    assert counters_after["live_allocations"] == counters_before["live_allocations"]
    assert counters_after["device_bytes"] <= counters_before["device_bytes"]
    gpu.close()
    backend.set_gemm_precision(-1)
    backend.disable()
