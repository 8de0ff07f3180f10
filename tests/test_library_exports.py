"""The C-ABI library loads without a GPU (and without the host program) and
exports every function its public header declares.  No compute is called."""
import ctypes
import os
import re

from conftest import PACKAGE, REPO


def declared_functions():
    text = ""
    for header in ("vitb200.h", "vitb200_augmentation.h"):
        text += open(os.path.join(REPO, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:cuda_backend|vitb200)_\w+)\s*\(", text)
    return sorted(set(names))


def test_every_declared_symbol_is_exported():
    library = os.path.join(PACKAGE, "libvitb200.so")
    assert os.path.exists(library), "run `python transformer-in-c_b200/build.py`"
    lib = ctypes.CDLL(library)
    names = declared_functions()
    assert len(names) >= 5 + 4 + 11
    for name in ("vitb200_data_augmentation_apply",
                 "vitb200_data_augmentation_translate",
                 "vitb200_data_augmentation_enabled"):
        assert name in names
    for name in ("cuda_backend_create", "cuda_backend_free",
                 "cuda_backend_available",
                 "cuda_backend_enable_device_execution",
                 "cuda_backend_disable_device_execution"):
        assert name in names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_create_reports_no_device_softly_without_gpu():
    """Reference contract (src/cuda_backend.cu:2021-2032): 1 = no usable
    device, and the output pointer is cleared."""
    import torch
    if torch.cuda.is_available():
        return
    lib = ctypes.CDLL(os.path.join(PACKAGE, "libvitb200.so"))
    handle = ctypes.c_void_p(1234)
    assert lib.cuda_backend_create(ctypes.byref(handle)) == 1
    assert handle.value is None
    assert lib.cuda_backend_available(None) == 0
    lib.cuda_backend_free(None)  # NULL-safe
    assert lib.cuda_backend_create(None) == -1
