"""The device-resident dataset against the reference's host pipeline
(vision_dataset_load_pgm_csv -> compute_pixel_statistics -> normalize_dataset
-> shuffle_dataset -> batch slices; tests/dataset_reference.py runs it in a
child process).  Every float a batch holds must be bit-identical to the float
the reference's dataset holds at that place: the kernel converts and
normalises with the same three roundings, and the shuffle is integer
arithmetic on the same draws."""
import numpy as np
import pytest

import dataset_reference as reference

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not reference.available(),
                                 reason="oracle/_ref/libtrainer_pieces.so not built")]


@pytest.mark.parametrize("samples,height,width,wide", [
    (37, 28, 28, False),   # 8-bit storage, four pixels per thread
    (19, 5, 7, False),     # odd image size: one pixel per thread
    (11, 6, 4, True),      # 16-bit storage
])
def test_batches_equal_the_reference_pipeline(vit_host_module, backend, tmp_path,
                                              samples, height, width, wide):
    manifest, _, _, labels = reference.write_dataset(tmp_path, samples, height,
                                                     width, seed=11, wide=wide)
    expected = reference.run(manifest, tmp_path, shuffles=2, state=977)
    launches = backend.kernel_launches()
    dataset = vit_host_module.Dataset(backend, manifest_path=manifest)
    assert (dataset.samples, dataset.height, dataset.width) == (samples, height, width)
    mean, inverse = dataset.statistics()
    assert np.float32(mean) == expected["mean"]
    assert np.float32(inverse) == expected["inverse_std"]

    # The loader's own values, then the normalised ones, in loaded order.
    status, images, got_labels = dataset.batch(0, samples, 0.0, 1.0)
    assert status == 0
    np.testing.assert_array_equal(images, expected["loaded"])
    np.testing.assert_array_equal(got_labels, labels)
    status, images, _ = dataset.batch(0, samples, mean, inverse)
    np.testing.assert_array_equal(images, expected["normalized"])

    state = 977
    for index in range(2):
        state = dataset.shuffle(state)
        assert state == int(expected["states"][index])
        want = expected[f"shuffled_{index}"]
        want_labels = expected[f"shuffled_labels_{index}"]
        batch = 8
        for offset in range(0, samples, batch):
            size = min(batch, samples - offset)
            status, images, got_labels = dataset.batch(offset, size, mean, inverse)
            assert status == 0
            np.testing.assert_array_equal(images, want[offset:offset + size])
            np.testing.assert_array_equal(got_labels, want_labels[offset:offset + size])
    assert backend.kernel_launches() > launches
    # Ranges that leave the dataset, and empty ones, are refused.
    assert dataset.batch(samples - 1, 2, mean, inverse)[0] == -1
    assert dataset.batch(samples + 1, 1, mean, inverse)[0] == -1
    assert dataset.batch(0, 0, mean, inverse)[0] == -1
    dataset.close()


def test_rejected_inputs_leave_no_dataset(vit_host_module, backend, tmp_path):
    with pytest.raises(RuntimeError):
        vit_host_module.Dataset(backend, manifest_path=str(tmp_path / "absent.csv"))
    with pytest.raises(RuntimeError):
        vit_host_module.Dataset(backend, pixels=np.zeros((2, 3, 3), np.uint16),
                                max_values=np.array([255, 0], np.uint16),
                                labels=np.zeros(2, np.uintp))


def test_batch_written_into_the_models_image_tensor(vit_host_module, host_lib,
                                                    backend, tmp_path):
    """The trainer's hand-over without a host round trip of our making: the
    batch kernel fills the cache's image tensor where it lives on the device
    and the forward pass reads it there.  (The reference's ops_upload_values
    still copies the tensor onto itself; its values survive that.)"""
    vh = vit_host_module
    config, batch = (1, 28, 28, 4, 32, 4, 2, 11), 6
    rng = np.random.RandomState(2)
    pixels = rng.randint(0, 256, size=(20, 28, 28)).astype(np.uint16)
    labels = rng.randint(0, 11, size=20).astype(np.uintp)
    backend.enable()
    backend.set_gemm_precision(1)
    dataset = vh.Dataset(backend, pixels=pixels, labels=labels)
    mean, inverse = dataset.statistics()
    dataset.shuffle(5)
    model = vh.VitHost(host_lib, config, batch)
    status, on_host, _ = dataset.batch(3, batch, mean, inverse)
    assert status == 0
    before = backend.memory_counters()
    status, _, got = dataset.batch(3, batch, mean, inverse,
                                   destination=model.images_tensor())
    assert status == 0
    after = backend.memory_counters()
    assert after["h2d_bytes"] == before["h2d_bytes"]   # nothing went up for it
    from_device = model.forward_from_address(model.images_tensor())
    from_host = model.forward(on_host)
    np.testing.assert_array_equal(from_device, from_host)
    backend.set_gemm_precision(-1)
    model.close()
    dataset.close()
    backend.disable()
