"""MDCI on two real GPUs in one process (the reference's mode, core.py:110-157):
shards on different devices, results gathered to devices[0] and merged there."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests import cases

pytestmark = pytest.mark.gpu


def test_mdci_two_devices_matches_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from dciknn_cuda_b200 import MDCI
    rng = np.random.default_rng(21)
    data = cases.latent_linear(rng, 20001, 16, 64, 0.01)
    query = cases.latent_linear(rng, 50, 16, 64, 0.01)
    projs = [cases.unit_rows(rng, 10, 64) for _ in range(2)]
    m = MDCI(64, 2, 5, 10, 10, devices=[0, 1], projs=[torch.from_numpy(p) for p in projs])
    m.add(torch.from_numpy(data))
    ids, dists = m.query(torch.from_numpy(query).cuda(0), 10, return_int_ids=True)
    assert ids.device.index == 0
    o = oracle.OracleMDCI(64, 2, 5, 10, 10, projs)
    o.add(data)
    oi, od = o.query(query, 10)
    assert np.array_equal(ids.cpu().numpy(), oi)
    assert np.array_equal(dists.cpu().numpy().view(np.uint32), od.view(np.uint32))
