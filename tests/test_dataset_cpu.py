"""Host side of the device-resident dataset (no GPU): the PGM + CSV parser, the
index-table shuffle and the pixel statistics against the reference's own
loader and trainer code (tests/dataset_reference.py runs them in a child
process).  Bit-exact: integers in, the loader's floats are value / max in one
rounding, and the shuffle is integer arithmetic."""
import ctypes
import os

import numpy as np
import pytest

import dataset_reference as reference

pytestmark = pytest.mark.skipif(not reference.available(),
                                reason="oracle/_ref/libtrainer_pieces.so not built")


@pytest.fixture(scope="module")
def lib(vit_host_module):
    return vit_host_module.load_backend_library()


@pytest.mark.parametrize("height,width,wide", [(28, 28, False), (5, 7, False),
                                               (6, 4, True)])
def test_parser_reads_what_the_reference_loader_reads(vit_host_module, lib,
                                                      tmp_path, height, width,
                                                      wide):
    manifest, pixels, maxima, labels = reference.write_dataset(
        tmp_path, 13, height, width, seed=3, wide=wide)
    expected = reference.run(manifest, tmp_path)
    assert int(expected["status"]) == 0
    status, ours, our_maxima, our_labels = vit_host_module.parse_pgm_csv(lib, manifest)
    assert status == 0
    np.testing.assert_array_equal(ours, pixels)
    np.testing.assert_array_equal(our_maxima, maxima)
    np.testing.assert_array_equal(our_labels, labels)
    np.testing.assert_array_equal(our_labels, expected["labels"])
    assert ours.shape[1:] == (int(expected["height"]), int(expected["width"]))
    floats = (ours.astype(np.float32) /
              our_maxima.astype(np.float32)[:, None, None]).reshape(len(ours), -1)
    np.testing.assert_array_equal(floats, expected["loaded"])


def _manifest(tmp_path, body):
    path = os.path.join(str(tmp_path), "manifest.csv")
    with open(path, "w") as handle:
        handle.write(body)
    return path


def _cases(tmp_path):
    """(name, manifest text) for inputs the reference loader rejects, plus a
    few odd ones it accepts."""
    good = os.path.join(str(tmp_path), "good.pgm")
    reference.write_pgm(good, np.arange(12).reshape(3, 4), 255, binary=True)
    other = os.path.join(str(tmp_path), "other.pgm")
    reference.write_pgm(other, np.arange(12).reshape(4, 3), 255, binary=True)
    over = os.path.join(str(tmp_path), "over.pgm")
    reference.write_pgm(over, np.full((3, 4), 9), 7, binary=False)
    over_binary = os.path.join(str(tmp_path), "over_binary.pgm")
    reference.write_pgm(over_binary, np.full((3, 4), 9), 7, binary=True)
    short = os.path.join(str(tmp_path), "short.pgm")
    with open(short, "wb") as handle:
        handle.write(b"P5\n4 3\n255\n\x01\x02\x03")
    magic = os.path.join(str(tmp_path), "magic.pgm")
    with open(magic, "wb") as handle:
        handle.write(b"P6\n4 3\n255\n" + bytes(36))
    zero = os.path.join(str(tmp_path), "zero.pgm")
    with open(zero, "wb") as handle:
        handle.write(b"P2\n0 3\n255\n")
    comments = os.path.join(str(tmp_path), "comments.pgm")
    with open(comments, "wb") as handle:
        handle.write(b"P2 # magic\n# size\n4\t3\r\n#max\n15\n" +
                     b" ".join(str(i).encode() for i in range(12)) + b"\n")
    return [
        ("missing file", f"{good},1\n{tmp_path}/nowhere.pgm,2\n"),
        ("mixed sizes", f"{good},1\n{other},2\n"),
        ("text value above the maximum", f"{over},1\n"),
        ("binary value above the maximum", f"{over_binary},1\n"),
        ("truncated raster", f"{short},1\n"),
        ("unknown magic", f"{magic},1\n"),
        ("zero width", f"{zero},1\n"),
        ("no samples", "# nothing\n\n"),
        ("no label", f"{good}\n"),
        ("comments and blanks in the header", f"  {comments},3\n{good}, 4\n"),
    ]


def test_parser_accepts_and_rejects_what_the_reference_does(vit_host_module, lib,
                                                            tmp_path):
    outcomes = []
    for name, body in _cases(tmp_path):
        manifest = _manifest(tmp_path, body)
        expected = reference.run(manifest, tmp_path)
        status, ours, maxima, labels = vit_host_module.parse_pgm_csv(lib, manifest)
        assert (status == 0) == (int(expected["status"]) == 0), name
        outcomes.append(status)
        if status == 0:
            floats = (ours.astype(np.float32) /
                      maxima.astype(np.float32)[:, None, None]).reshape(len(ours), -1)
            np.testing.assert_array_equal(floats, expected["loaded"], err_msg=name)
            np.testing.assert_array_equal(labels, expected["labels"], err_msg=name)
    assert 0 in outcomes and -1 in outcomes
    assert vit_host_module.parse_pgm_csv(lib, str(tmp_path / "absent.csv"))[0] == -1


@pytest.mark.parametrize("samples", [1, 2, 37])
def test_index_shuffle_is_the_reference_shuffle(lib, tmp_path, samples):
    """The reference moves images; a sample's first pixel tells which one it
    is.  Three shuffles in a row, continuing the generator state."""
    manifest, pixels, _, _ = reference.write_dataset(tmp_path, samples, 2, 2, seed=5)
    expected = reference.run(manifest, tmp_path, shuffles=3, state=20240229)
    loaded = expected["loaded"]
    order = np.arange(samples, dtype=np.uint32)
    state = ctypes.c_ulong(20240229)
    for index in range(3):
        lib.vitb200_dataset_shuffle_order(
            order.ctypes.data_as(ctypes.POINTER(ctypes.c_uint)), samples,
            ctypes.byref(state))
        assert sorted(order) == list(range(samples))
        assert int(state.value) == int(expected["states"][index])
        # The reference only normalised and moved the samples.
        moved = expected[f"shuffled_{index}"]
        np.testing.assert_array_equal(
            moved, expected["normalized"][order], err_msg=f"shuffle {index}")
    assert loaded.shape[0] == samples


def test_pixel_statistics_are_the_trainers(lib, tmp_path):
    manifest, pixels, maxima, _ = reference.write_dataset(tmp_path, 29, 9, 5, seed=8)
    expected = reference.run(manifest, tmp_path)
    mean, inverse = ctypes.c_float(), ctypes.c_float()
    ushort_p = ctypes.POINTER(ctypes.c_ushort)
    flat = np.ascontiguousarray(pixels.reshape(len(pixels), -1))
    assert lib.vitb200_dataset_pixel_statistics(
        flat.ctypes.data_as(ushort_p), maxima.ctypes.data_as(ushort_p),
        len(pixels), flat.shape[1], ctypes.byref(mean), ctypes.byref(inverse)) == 0
    assert np.float32(mean.value) == expected["mean"]
    assert np.float32(inverse.value) == expected["inverse_std"]
