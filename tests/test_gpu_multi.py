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


def _nccl_worker(rank, world, port, out_dir):
    import os
    import sys
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from dciknn_cuda_b200 import MDCI
    rng = np.random.default_rng(33)
    data = cases.latent_linear(rng, 12001, 16, 64, 0.01)
    query = cases.latent_linear(rng, 40, 16, 64, 0.01)
    projs = [cases.unit_rows(rng, 10, 64) for _ in range(world)]
    m = MDCI(64, 2, 5, 10, 10, process_group=dist.group.WORLD, projs=[torch.from_numpy(p) for p in projs])
    m.add(torch.from_numpy(data))
    ids, dists = m.query(torch.from_numpy(query), 10, return_int_ids=True)
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), ids=ids.cpu().numpy(), dists=dists.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_mdci_one_process_per_gpu_over_nccl(tmp_path):
    """MDCI(process_group=...): two ranks, two GPUs, NCCL all-gather of the per-shard lists and
    the device merge; every rank must end with the reference MDCI's merged result."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os
    import torch.multiprocessing as mp
    world, port = 2, 29600 + os.getpid() % 300
    mp.spawn(_nccl_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(33)
    data = cases.latent_linear(rng, 12001, 16, 64, 0.01)
    query = cases.latent_linear(rng, 40, 16, 64, 0.01)
    projs = [cases.unit_rows(rng, 10, 64) for _ in range(world)]
    o = oracle.OracleMDCI(64, 2, 5, 10, 10, projs)
    o.add(data)
    oi, od = o.query(query, 10)
    for r in range(world):
        z = np.load(os.path.join(str(tmp_path), "rank%d.npz" % r))
        assert np.array_equal(z["ids"], oi)
        assert np.array_equal(z["dists"].view(np.uint32), od.view(np.uint32))
