"""ctypes driver for the reference project's own CUDA build (TEST INFRASTRUCTURE ONLY).

Loads oracle/_ref/libdci_ref.so (or the race-fixed variant), which
oracle/build_ref.py compiles from the reference's unmodified sources plus
oracle/ref_harness.cu.  Needs a GPU.  Device memory comes from torch tensors.
libcublas must already be loaded, so torch is imported first.
"""
import ctypes as C
import os

import numpy as np
import torch

from .build_ref import REF_FIXED_SO, REF_SO


def available(race_fixed=False):
    return os.path.exists(REF_FIXED_SO if race_fixed else REF_SO) and torch.cuda.is_available()


class ReferenceDCI:
    """The reference's dci_* C API (include/dci.h:58-84) behind the harness."""

    def __init__(self, dim, L, S, bs=100, ts=10, device=0, race_fixed=False):
        torch.zeros(1, device="cuda:%d" % device) @ torch.zeros(1, device="cuda:%d" % device)   # loads cuBLAS
        self.lib = C.CDLL(REF_FIXED_SO if race_fixed else REF_SO, mode=C.RTLD_LOCAL)
        self.lib.ref_last_error.restype = C.c_char_p
        self.dim, self.L, self.S, self.P, self.T, self.device = dim, L, S, bs, ts, device
        self.h = C.c_void_p()
        self._ck(self.lib.ref_dci_create(C.byref(self.h), dim, L, S, device))
        self.N = 0
        self._data = None

    def _ck(self, rc):
        if rc != 0:
            raise RuntimeError("reference harness: " + self.lib.ref_last_error().decode())

    def get_proj(self):
        out = np.empty((self.L * self.S, self.dim), np.float32)
        self._ck(self.lib.ref_dci_get_proj(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    def set_proj(self, proj):
        proj = np.ascontiguousarray(proj, np.float32)
        assert proj.shape == (self.L * self.S, self.dim)
        self._ck(self.lib.ref_dci_set_proj(self.h, proj.ctypes.data_as(C.c_void_p)))

    def add(self, data):
        assert data.is_cuda and data.dtype == torch.float32 and data.is_contiguous()
        self._data = data
        self.N = data.shape[0]
        torch.cuda.synchronize()
        self._ck(self.lib.ref_dci_add(self.h, self.N, C.c_void_p(data.data_ptr()), self.P, self.T))

    def get_index(self):
        I = self.L * self.S
        keys = np.empty((I, self.N), np.float32)
        ids = np.empty((I, self.N), np.int32)
        self._ck(self.lib.ref_dci_get_index(self.h, keys.ctypes.data_as(C.c_void_p), ids.ctypes.data_as(C.c_void_p)))
        return keys, ids

    def project_queries(self, query):
        """[nq][I] projected queries computed by the reference's own cuBLAS call."""
        out = np.empty((query.shape[0], self.L * self.S), np.float32)
        torch.cuda.synchronize()
        self._ck(self.lib.ref_dci_project_queries(self.h, query.shape[0], C.c_void_p(query.data_ptr()),
                                                  out.ctypes.data_as(C.c_void_p)))
        return out

    def query(self, query, k, num_outer_iterations=5000, max_num_candidates=None):
        assert query.is_cuda and query.dtype == torch.float32 and query.is_contiguous()
        mc = 10 * k if max_num_candidates is None else max_num_candidates
        ids = torch.empty((query.shape[0], k), dtype=torch.int32, device=query.device)
        dists = torch.empty((query.shape[0], k), dtype=torch.float32, device=query.device)
        torch.cuda.synchronize()
        self._ck(self.lib.ref_dci_query(self.h, query.shape[0], C.c_void_p(query.data_ptr()), k,
                                        int(num_outer_iterations), int(mc), self.P, self.T,
                                        C.c_void_p(ids.data_ptr()), C.c_void_p(dists.data_ptr())))
        return ids, dists

    def clear(self):
        self._ck(self.lib.ref_dci_clear(self.h))
        self.N = 0
        self._data = None

    def free(self):
        if self.h:
            self.lib.ref_dci_destroy(self.h)
            self.h = C.c_void_p()
