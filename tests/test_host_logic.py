"""Host-side logic that needs no GPU: workload shaping."""
import torch

import __graft_entry__ as entry


def test_zipf_target_is_a_capped_distribution():
    entry.load_package()
    from p92moe_b200 import synth

    for alpha in (1.0, 1.2):
        share = synth.zipf_target(alpha, seed=3)
        assert abs(float(share.sum()) - 1.0) < 1e-4
        assert float(share.max()) <= 1.0 / 8 + 1e-6
        ranked = torch.sort(share, descending=True).values
        assert ranked[0] >= ranked[10] >= ranked[100] > 0
    a = synth.zipf_target(1.2, seed=3)
    b = synth.zipf_target(1.2, seed=4)
    assert not torch.equal(a, b) and torch.allclose(torch.sort(a).values, torch.sort(b).values)
