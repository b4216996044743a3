"""Parameter search for a recall target, on the device."""
import numpy as np
import pytest
import torch

import cases
from dciknn_cuda_b200 import DCI, tuning
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_tune_returns_the_fastest_parameter_set_that_reaches_the_target():
    rng = np.random.default_rng(5)
    data_h = cases.latent_linear(rng, 30000, 8, 32, 0.01)
    query_h = cases.latent_linear(rng, 256, 8, 32, 0.01)
    data, query = torch.from_numpy(data_h).cuda(), torch.from_numpy(query_h).cuda()
    truth = tuning.exact_neighbours(data, query, 10)
    bi, _ = oracle.bruteforce(data_h, query_h, 10)
    assert tuning.recall(torch.from_numpy(bi), truth.cpu()) > 0.999      # ground truth itself
    grid = [tuning.Params(2, 7, 100, 10, 5000, 100), tuning.Params(1, 3, 20, 10, 5000, 20),
            tuning.Params(2, 5, 50, 10, 5000, 50), tuning.Params(1, 7, 100, 20, 5000, 100)]
    seen = []
    best, trials = tuning.tune(data, query, 10, 0.9, grid=grid, seed=9, progress=seen.append)
    assert len(trials) == len(grid) == len(seen)
    feasible = [t for t in trials if t.recall >= 0.9]
    assert feasible, [t.as_dict() for t in trials]
    assert best.feasible and best.queries_per_s == max(t.queries_per_s for t in feasible)
    # the reported recall is what a user gets with those parameters and the same seed
    p = best.params
    dci = DCI(32, p.num_comp_indices, p.num_simp_indices, p.bs, p.ts, seed=9)
    dci.add(data)
    ids, _ = dci.query(query, 10, p.num_outer_iterations, max_num_candidates=p.max_num_candidates, return_int_ids=True)
    assert tuning.recall(ids, truth) == pytest.approx(best.recall)
    dci.free()


def test_tune_without_a_feasible_set_returns_the_best_recall():
    rng = np.random.default_rng(6)
    data = torch.from_numpy(cases.latent_linear(rng, 8000, 8, 32, 0.01)).cuda()
    query = torch.from_numpy(cases.latent_linear(rng, 64, 8, 32, 0.01)).cuda()
    grid = [tuning.Params(1, 3, 10, 10, 5000, 10), tuning.Params(1, 3, 10, 10, 5000, 20)]
    best, trials = tuning.tune(data, query, 10, 1.0, grid=grid)
    assert not best.feasible and best.recall == max(t.recall for t in trials)
