"""The reference's own dataset pipeline, as the checker of the device-resident
dataset: vision_dataset_load_pgm_csv (reference src/dataset.c:136-226) followed
by the trainer's compute_pixel_statistics, normalize_dataset and
shuffle_dataset (reference examples/organ_smnist.c:75-139), all compiled from
the reference's sources into oracle/_ref/libtrainer_pieces.so.

That library carries its own copy of the reference's host code, so it is run
in a process of its own (`python dataset_reference.py manifest out.npz
shuffles state`) and never loaded next to the host library the backend binds
to.  Also here: a writer of small PGM files in every dialect the loader reads.
"""
import ctypes
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY = os.path.join(os.path.dirname(HERE), "oracle", "_ref",
                       "libtrainer_pieces.so")


class VisionDataset(ctypes.Structure):
    """Layout of the reference's VisionDataset (include/dataset.h:6-13)."""
    _fields_ = [("images", ctypes.POINTER(ctypes.c_float)),
                ("labels", ctypes.POINTER(ctypes.c_size_t)),
                ("sample_count", ctypes.c_size_t), ("height", ctypes.c_size_t),
                ("width", ctypes.c_size_t), ("channels", ctypes.c_size_t)]


def available():
    return os.path.exists(LIBRARY)


def _snapshot(dataset):
    count = dataset.sample_count * dataset.height * dataset.width
    images = np.ctypeslib.as_array(dataset.images, shape=(count,)).copy()
    labels = np.ctypeslib.as_array(dataset.labels,
                                   shape=(dataset.sample_count,)).copy()
    return images.reshape(dataset.sample_count, -1), labels


def _child(manifest, output, shuffles, state):
    lib = ctypes.CDLL(LIBRARY)
    dataset = VisionDataset()
    status = lib.vision_dataset_load_pgm_csv(os.fsencode(manifest),
                                             ctypes.byref(dataset))
    result = {"status": np.int64(status)}
    if status == 0:
        result["height"] = np.int64(dataset.height)
        result["width"] = np.int64(dataset.width)
        result["loaded"], result["labels"] = _snapshot(dataset)
        mean, inverse = ctypes.c_float(), ctypes.c_float()
        lib.trainer_statistics(ctypes.byref(dataset), ctypes.byref(mean),
                               ctypes.byref(inverse))
        result["mean"] = np.float32(mean.value)
        result["inverse_std"] = np.float32(inverse.value)
        lib.trainer_normalize.argtypes = [ctypes.c_void_p, ctypes.c_float,
                                          ctypes.c_float]
        lib.trainer_normalize(ctypes.byref(dataset), mean, inverse)
        result["normalized"], _ = _snapshot(dataset)
        generator = ctypes.c_ulong(state)
        states = []
        for index in range(shuffles):
            lib.trainer_shuffle(ctypes.byref(dataset), ctypes.byref(generator))
            images, labels = _snapshot(dataset)
            result[f"shuffled_{index}"] = images
            result[f"shuffled_labels_{index}"] = labels
            states.append(generator.value)
        result["states"] = np.array(states, dtype=np.uint64)
        lib.vision_dataset_free(ctypes.byref(dataset))
    np.savez(output, **result)


def run(manifest, directory, shuffles=0, state=1):
    """Runs the reference pipeline on `manifest` in a child process (with the
    manifest's directory as working directory, like the loader's relative
    paths expect) and returns the saved arrays."""
    output = os.path.join(str(directory), "reference_dataset.npz")
    subprocess.run([sys.executable, os.path.abspath(__file__), str(manifest),
                    output, str(shuffles), str(state)], check=True,
                   cwd=os.path.dirname(os.path.abspath(str(manifest))), timeout=300)
    return dict(np.load(output))


def _time_child(samples, height, width):
    """Seconds the reference's trainer spends per epoch on a dataset that is
    already in memory: shuffle_dataset (images moved by memcpy); and once per
    run: normalize_dataset."""
    import json
    import time
    lib = ctypes.CDLL(LIBRARY)
    rng = np.random.RandomState(1)
    images = rng.rand(samples, height * width).astype(np.float32)
    labels = rng.randint(0, 11, size=samples).astype(np.uintp)
    dataset = VisionDataset(
        images.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
        labels.ctypes.data_as(ctypes.POINTER(ctypes.c_size_t)), samples, height,
        width, 1)
    lib.trainer_normalize.argtypes = [ctypes.c_void_p, ctypes.c_float,
                                      ctypes.c_float]
    start = time.perf_counter()
    lib.trainer_normalize(ctypes.byref(dataset), 0.5, 2.0)
    normalise = time.perf_counter() - start
    state = ctypes.c_ulong(1)
    lib.trainer_shuffle(ctypes.byref(dataset), ctypes.byref(state))
    start = time.perf_counter()
    for _ in range(3):
        lib.trainer_shuffle(ctypes.byref(dataset), ctypes.byref(state))
    shuffle = (time.perf_counter() - start) / 3
    print(json.dumps({"shuffle_seconds": shuffle, "normalise_seconds": normalise}))


def time_reference(samples, height, width):
    """Runs _time_child in a process of its own; None if the library is absent."""
    import json
    if not available():
        return None
    done = subprocess.run([sys.executable, os.path.abspath(__file__), "time",
                           str(samples), str(height), str(width)],
                          capture_output=True, text=True, timeout=300)
    if done.returncode != 0:
        return None
    return json.loads(done.stdout.strip().splitlines()[-1])


def write_pgm(path, pixels, max_value, binary, comment=False):
    """One PGM file: P5 (binary; two bytes per sample, most significant first,
    when max_value >= 256) or P2 (decimal text)."""
    height, width = pixels.shape
    note = "# a comment line\n" if comment else ""
    header = f"{'P5' if binary else 'P2'}\n{note}{width} {height}\n{max_value}\n"
    with open(path, "wb") as handle:
        handle.write(header.encode())
        if binary:
            kind = ">u2" if max_value >= 256 else "u1"
            handle.write(pixels.astype(kind).tobytes())
        else:
            rows = [" ".join(str(int(v)) for v in row) for row in pixels]
            handle.write(("\n".join(rows) + "\n").encode())


def write_dataset(directory, samples, height, width, seed, wide=False):
    """A manifest with `samples` images that cycle through the dialects: P5
    and P2, with and without a comment, differing maximum values.  Returns
    (manifest path, pixels [samples, height, width], max values, labels)."""
    rng = np.random.RandomState(seed)
    directory = str(directory)
    lines = ["# manifest written by tests/dataset_reference.py", ""]
    pixels = np.zeros((samples, height, width), np.uint16)
    maxima = np.zeros(samples, np.uint16)
    labels = rng.randint(0, 11, size=samples)
    for index in range(samples):
        if wide:
            maximum = [65535, 1023, 255, 4095][index % 4]
        else:
            maximum = [255, 255, 200, 15][index % 4]
        pixels[index] = rng.randint(0, maximum + 1, size=(height, width))
        maxima[index] = maximum
        name = f"image_{index:04d}.pgm"
        write_pgm(os.path.join(directory, name), pixels[index], maximum,
                  binary=index % 3 != 1, comment=index % 5 == 2)
        lines.append(f"{os.path.join(directory, name)},{labels[index]}")
    manifest = os.path.join(directory, "manifest.csv")
    with open(manifest, "w") as handle:
        handle.write("\n".join(lines) + "\n")
    return manifest, pixels, maxima, labels.astype(np.uintp)


if __name__ == "__main__":
    if sys.argv[1] == "time":
        _time_child(int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]))
    else:
        _child(sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]))
