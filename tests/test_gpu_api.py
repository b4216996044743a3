"""The DCI class must reject what the reference's Python layer rejects, with the
same exception types (dciknn_cuda/core.py:53-71, 78-92, 131-132), and clear /
reset must behave like dci_clear / dci_reset (dci_cuda_kernel.cu:878-891)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk():
    from dciknn_cuda_b200 import DCI
    return DCI(16, 2, 3, 4, 5, seed=1)


def test_argument_checks_follow_the_reference():
    g = _mk()
    good = torch.randn(50, 16, device="cuda")
    with pytest.raises(ValueError):
        g.add(torch.randn(50, 15, device="cuda"))
    with pytest.raises(TypeError):
        g.add(good.double())
    with pytest.raises(ValueError):
        g.add(torch.randn(16, 50, device="cuda").t())
    with pytest.raises(TypeError):
        g.add(good.cpu())
    g.add(good)
    assert g.num_points == 50
    with pytest.raises(RuntimeError):
        g.add(good)
    with pytest.raises(TypeError):
        g.query(good[:2], 2.0)
    with pytest.raises(ValueError):
        g.query(good[:2], 0)
    with pytest.raises(ValueError):
        g.query(good[:2], 51)
    bi, bw = g.query(good[:2], 3, blind=True)      # candidates in retrieval order, width min(5000, 10 * 3)
    assert bi.shape == bw.shape == (2, 30)
    ids, dists = g.query(good[:3])          # num_neighbours = -1 means all points (core.py:84-85)
    assert ids.shape == (3, 50) and bool((dists[:, 1:] >= dists[:, :-1]).all())
    assert torch.equal(ids[:, 0].long().cpu(), torch.arange(3))   # a point is its own nearest neighbour


def test_clear_keeps_directions_and_reset_redraws_them():
    g = _mk()
    p0 = g.get_proj()
    x = torch.randn(40, 16, device="cuda")
    g.add(x)
    with pytest.raises(RuntimeError):
        g.set_proj(p0)
    g.clear()
    assert g.num_points == 0 and torch.equal(g.get_proj(), p0)
    with pytest.raises(RuntimeError):
        g.query(x[:1], 1)
    g.add(x)
    a = g.query(x[:4], 3)
    g.reset()
    assert not torch.equal(g.get_proj(), p0) and g.num_points == 0
    g.add(x)
    g.free()
    g.free()
    with pytest.raises(RuntimeError):
        g.add(x)
    assert a[0].shape == (4, 3)


def test_mdci_rejects_non_positive_k():
    from dciknn_cuda_b200 import MDCI
    m = MDCI(16, 2, 3, 4, 5, devices=[0])
    m.add(torch.randn(30, 16))
    with pytest.raises(RuntimeError):
        m.query(torch.randn(2, 16, device="cuda"), -1)
    ids, dists = m.query(torch.randn(2, 16, device="cuda"), 4)
    assert ids.shape == (2, 4) and ids.dtype == torch.float32
