"""The plain implementation against the logits that izmttk/ullm's own model
code produced on the CPU (tests/golden/make_golden.py made the files)."""

import os

import pytest
import torch

import plain_model as pm
from tiny_configs import ALL

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("tag", ["A", "B"])
def test_logits_match_reference_model_code(tag):
    cfg, init, _ = ALL[tag]
    gold = torch.load(os.path.join(GOLDEN, f"ref_logits_{tag}.pt"))
    w = pm.random_weights(cfg, **init)
    for ids, ref in zip(gold["prompts"], gold["logits"]):
        got = pm.forward_logits(ids, w, cfg)
        assert got.shape == ref.shape
        assert (got - ref).abs().max().item() <= 2e-6 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("tag", ["A", "B"])
def test_filtered_distribution_matches_reference_sampler(tag):
    gold = torch.load(os.path.join(GOLDEN, f"ref_logits_{tag}.pt"))
    for row, (t, k, p, mp), ref in zip(gold["sampler_logits"], gold["sampler_cases"], gold["sampler_dists"]):
        got = pm.filtered_distribution(row, t, k, p, mp)
        assert torch.equal(got > 0, ref > 0)
        assert (got - ref).abs().max().item() <= 1e-6


def test_whole_sequence_prefix_property():
    """Causality: logits of a prefix equal the prefix of the logits."""
    cfg, init, _ = ALL["C"]
    w = pm.random_weights(cfg, **init)
    ids = torch.randint(0, cfg["vocab_size"], (60,), generator=torch.Generator().manual_seed(5))
    full = pm.forward_logits(ids, w, cfg)
    part = pm.forward_logits(ids[:37], w, cfg)
    assert (full[:37] - part).abs().max().item() < 1e-5


def test_window_changes_far_positions_only():
    cfg, init, _ = ALL["C"]
    w = pm.random_weights(cfg, **init)
    ids = torch.randint(0, cfg["vocab_size"], (60,), generator=torch.Generator().manual_seed(6))
    nowin = dict(cfg, use_sliding_window=False)
    a = pm.forward_logits(ids, w, cfg)
    b = pm.forward_logits(ids, w, nowin)
    W = cfg["sliding_window"]
    assert (a[:W] - b[:W]).abs().max().item() < 1e-6
    assert (a[W:] - b[W:]).abs().max().item() > 1e-4
