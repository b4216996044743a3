"""CPU-side checks of the boundary: the shared library loads and exports every
symbol include/dci_b200.h declares; argument errors are reported without a GPU."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "dci_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dci_b200_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from dciknn_cuda_b200 import _capi
    from dciknn_cuda_b200.build import build
    build()
    lib = C.CDLL(_capi.LIB_PATH)
    names = _declared()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(n for n, _, _ in _capi.SYMBOLS) == names
    assert _capi.lib().dci_b200_abi_version() == 1


def test_argument_errors_need_no_gpu():
    from dciknn_cuda_b200 import _capi
    lib = _capi.lib()
    h = C.c_void_p()
    assert lib.dci_b200_create(C.byref(h), 0, 2, 3, 0, 1) == _capi.ERR_ARG
    assert b"dim" in lib.dci_b200_last_error()
    assert lib.dci_b200_create(C.byref(h), 8, 0, 3, 0, 1) == _capi.ERR_ARG
    assert lib.dci_b200_create(C.byref(h), 8, 100, 100, 0, 1) == _capi.ERR_UNSUPPORTED
    assert lib.dci_b200_add(None, None, 1, 1, 1, None) == _capi.ERR_ARG
    assert lib.dci_b200_query(None, None, 1, 1, 1, 1, 0, 1, 1, None, None, None) == _capi.ERR_ARG
    assert lib.dci_b200_destroy(None) == 0


def test_torch_shim_builds_and_exposes_the_reference_entry_points():
    """The PyTorch-extension module carries the seven functions of the reference's `_dci_cuda`
    (src/dci_cuda.cpp:175-183); without a GPU, creating an instance fails loudly."""
    import pytest
    import torch  # noqa: F401  (the module links against libtorch)
    from dciknn_cuda_b200.build import build_torch_shim
    build_torch_shim()
    from dciknn_cuda_b200 import _dci_b200
    for name in ("_dci_new", "_dci_add", "_dci_query", "_dci_multi_query", "_dci_clear", "_dci_reset", "_dci_free"):
        assert callable(getattr(_dci_b200, name)), name
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            _dci_b200._dci_new(8, 2, 3, 0)
