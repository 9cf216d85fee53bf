"""The row-sampled oracle used for CPU timing must compute the same rows as the full oracle."""
import torch

from oracle import pairformer_oracle as orc
from oracle import sampled
from tt_boltz_b200 import synthetic
from tests.conftest import rel_l2


def test_sampled_rows_equal_full_oracle():
    n = 20
    sd = synthetic.make_weights(1, seed=5, std=0.05, affine_jitter=0.3)
    s, z = synthetic.make_inputs(n, seed=4)
    g = torch.Generator().manual_seed(9)
    pm = (torch.rand(n, n, generator=g) > 0.2).float()
    rows = torch.tensor([1, 4, 5, 13, 19])
    z0 = z[0]
    pre = "layers.0."
    with torch.no_grad():
        for incoming, name in ((False, "tri_mul_out"), (True, "tri_mul_in")):
            full = z0 + orc.tri_mul(z0, sd, pre + name, pm, incoming)
            assert rel_l2(sampled.tri_mul_rows(z0, sd, pre + name, pm, incoming, rows)[0], full[rows]) < 1e-6
        full = z0 + orc.tri_att(z0, sd, pre + "tri_att_start", pm, False)
        assert rel_l2(sampled.tri_att_rows(z0, sd, pre + "tri_att_start", pm, False, rows)[0], full[rows]) < 1e-6
        full = z0 + orc.tri_att(z0, sd, pre + "tri_att_end", pm, True)
        assert rel_l2(sampled.tri_att_rows(z0, sd, pre + "tri_att_end", pm, True, rows)[0], full[:, rows].transpose(0, 1)) < 1e-6
        full = z0 + orc.transition(z0, sd, pre + "transition_z")
        assert rel_l2(sampled.transition_rows(z0, sd, pre + "transition_z", rows)[0], full[rows]) < 1e-6
        t = sampled.sampled_block_seconds(s[0], z0, torch.ones(n), pm, sd, pre, 5)
        assert t["total"] > 0 and set(t) >= {"tri_mul_out", "tri_att_end", "single_track"}
