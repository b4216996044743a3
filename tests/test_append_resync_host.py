"""Host logic of DCI.append when the library reports a failure: the Python object must follow the
handle (which a failed append may have emptied) instead of keeping its old counts.  Runs on CPU with
a stand-in for the C library."""
import contextlib
import ctypes as C

import pytest
import torch


class _StubLib:
    """dci_b200_append fails with a CUDA status and leaves the handle with `points_left` points."""

    def __init__(self, points_left):
        self.points_left = points_left

    def dci_b200_append(self, *args):
        return 3                                   # DCI_B200_ERR_CUDA

    def dci_b200_num_points(self, handle):
        return self.points_left

    def dci_b200_last_error(self):
        return b"cudaMalloc failed (stub)"

    def dci_b200_destroy(self, handle):
        return 0


@pytest.mark.parametrize("points_left", [0, 100])
def test_failed_append_resyncs_the_python_object(monkeypatch, points_left):
    from dciknn_cuda_b200 import _capi, core
    stub = _StubLib(points_left)
    monkeypatch.setattr(_capi, "lib", lambda: stub)
    monkeypatch.setattr(core.torch.cuda, "device", lambda idx: contextlib.nullcontext())
    monkeypatch.setattr(core, "_stream_ptr", lambda dev: C.c_void_p(0))
    g = object.__new__(core.DCI)
    g._dim, g._num_comp_indices, g._num_simp_indices = 4, 1, 2
    g._block_size, g._thread_size, g._device = 2, 2, None      # CPU tensors have no device index
    g._handle = C.c_void_p(1)
    g.num_points = 100
    g._array = torch.zeros(100, 4)
    g._store = None
    monkeypatch.setattr(g, "_check_data", lambda arr: None)
    with pytest.raises(_capi.DCIError):
        g.append(torch.ones(10, 4))
    assert g.num_points == points_left
    if points_left == 0:
        assert g._array is None and g._store is None
    else:
        assert g._array is not None and g._array.shape[0] == 100
    g._handle = C.c_void_p()                      # nothing to free
