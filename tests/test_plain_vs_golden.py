"""The plain implementation against logits made by the reference's own Python model (tests/golden/)."""
import os

import numpy as np
import pytest
import torch

from plain_qwen2 import PlainModel, causal_attention, causal_attention_fast
from tiny_configs import TINY_A, TINY_B

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name,cfg_json", [("A", TINY_A), ("B", TINY_B)])
def test_plain_matches_reference_model(name, cfg_json, tmp_path):
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    g = np.load(os.path.join(GOLDEN, f"qwen2_tiny_{name}.npz"))
    d = str(tmp_path / "m")
    write_random_model(config_from_json_dict(cfg_json), d, seed=int(g["seed"]), dtype="float32")
    plain = PlainModel(d, torch.float64)
    for i in range(3):
        ids = g[f"ids{i}"].tolist()
        want = torch.from_numpy(g[f"logits{i}"]).double()
        got = plain.logits(ids)
        assert not torch.isnan(got).any()
        # The reference's Python model computes in float32 with float32 rotation angles.
        assert (got - want).abs().max().item() < 2e-5
        assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_attention_loop_equals_masked():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(19, 6, 8, generator=g, dtype=torch.float64)
    k = torch.randn(19, 2, 8, generator=g, dtype=torch.float64)
    v = torch.randn(19, 2, 8, generator=g, dtype=torch.float64)
    for window in (0, 5):
        a, b = causal_attention(q, k, v, window), causal_attention_fast(q, k, v, window)
        assert (a - b).abs().max().item() < 1e-12


def test_plain_is_causal(tmp_path):
    from nanoinfer_b200.registry import config_from_json_dict
    from nanoinfer_b200.weights import write_random_model
    d = str(tmp_path / "m")
    write_random_model(config_from_json_dict(TINY_A), d, seed=5)
    plain = PlainModel(d)
    ids = list(range(3, 20))
    a = plain.logits(ids)
    ids2 = ids[:-1] + [200]
    b = plain.logits(ids2)
    assert torch.equal(a[:-1], b[:-1]) and not torch.equal(a[-1], b[-1])
    assert (plain.logits(ids[:9]) - a[:9]).abs().max().item() < 1e-12
