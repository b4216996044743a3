"""Host logic of the parameter search (no GPU): grid, recall scoring, selection, budget."""
import pytest
import torch

from dciknn_cuda_b200 import tuning


def test_recall_counts_set_overlap_per_query():
    truth = torch.tensor([[1, 2, 3, 4], [5, 6, 7, 8]])
    ids = torch.tensor([[4, 3, 9, 1], [0, 0, 0, 5]])
    assert tuning.recall(ids, truth) == pytest.approx((3 + 1) / 8)
    assert tuning.recall(truth.flip(1), truth) == 1.0


def test_default_grid_keeps_partitions_large_enough():
    g = tuning.default_grid(10, 20_000)
    assert g and all(-(-20_000 // p.bs) >= 40 for p in g)
    assert any(p.bs == 400 for p in g) and not any(p.bs == 1000 for p in g)
    assert tuning.Params(2, 7, 100, 10, 5000, 100) in g         # the reference's defaults


def _trial(recall, qps, **kw):
    return tuning.Trial(tuning.Params(**kw), recall, qps, 1.0)


def test_select_prefers_fastest_feasible_then_best_recall():
    a, b, c = _trial(0.95, 10.0), _trial(0.91, 30.0, bs=50), _trial(0.5, 99.0, bs=25)
    assert tuning.select([a, b, c], 0.9) is b
    assert [t.feasible for t in (a, b, c)] == [True, True, False]
    assert tuning.select([a, b, c], 0.99) is a                   # nothing reaches 0.99
    assert tuning.select([], 0.9) is None


def test_tune_skips_rejected_parameter_sets_and_honours_budget():
    calls = []

    def fake_measure(data, q, truth, k, p, device, seed=1, repeats=2):
        calls.append(p)
        if p.num_simp_indices == 5:
            raise ValueError("rejected")
        return tuning.Trial(p, 0.8 + 0.01 * p.num_simp_indices, 1000.0 / p.num_simp_indices, 1.0)

    class FakeCuda(torch.Tensor):
        is_cuda = True
        device = torch.device("cuda", 0)

    data = torch.zeros(100, 4).as_subclass(FakeCuda)
    grid = [tuning.Params(num_simp_indices=s) for s in (3, 5, 10, 12)]
    best, trials = tuning.tune(data, torch.zeros(8, 4), 2, 0.9, grid=grid, truth=torch.zeros(8, 2),
                               measure_fn=fake_measure)
    assert len(calls) == 4 and len(trials) == 3
    assert best.params.num_simp_indices == 10
    calls.clear()
    best, trials = tuning.tune(data, torch.zeros(8, 4), 2, 0.9, grid=grid, truth=torch.zeros(8, 2),
                               budget_s=0.0, measure_fn=fake_measure)
    assert 1 <= len(trials) <= 2                                 # stops after the first finished trial
    with pytest.raises(TypeError):
        tuning.tune(torch.zeros(4, 4), torch.zeros(1, 4), 2)
    with pytest.raises(ValueError):
        tuning.tune(data, torch.zeros(1, 4), 2, target_recall=0.0)
