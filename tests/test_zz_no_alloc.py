"""The allocation-free triangle-multiplication entry point.

Some hosts of this library cannot hand it scratch memory: they run inside a fixed device-memory
budget, or call from a place where the allocator must not be entered, or forbid allocation once
serving has started.  ``b200pf_tri_mul_noalloc`` keeps its intermediate planes in an array that
is part of the library image instead.  This test drives it through the C ABI, twice in a row
(the array is shared and keeps the previous call's contents), and checks the result against the
ordinary producer / contraction / epilogue entry points fed with caller-owned planes.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import pytest
import torch

from tt_boltz_b200 import _lib, ops, synthetic, weights
from tt_boltz_b200._lib import call, ptr, stream

pytestmark = pytest.mark.gpu


def _strip(sd):
    return {k[len("layers.0."):]: v for k, v in sd.items()}


def test_noalloc_matches_stage_entry_points_twice_in_a_row():
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    sd = _strip(synthetic.make_weights(1, seed=5, std=0.05, affine_jitter=0.3, with_s=False))
    for call_no, (n, incoming, seed) in enumerate([(100, False, 4), (72, True, 6)]):
        _, z = synthetic.make_inputs(n, seed=seed, with_s=False)
        g = torch.Generator().manual_seed(seed)
        pm = (torch.rand(n, n, generator=g) > 0.2).to(torch.uint8).to(dev)
        pre = "tri_mul_in." if incoming else "tri_mul_out."
        w = weights.pack_trimul(sd, pre, dev)
        z_ref = z[0].to(dev).clone()
        ops.tri_mul_bf16(z_ref, pm, w, ops.Workspace(n, dev), incoming)
        z_new = z[0].to(dev).clone()
        before = torch.cuda.memory_allocated(dev)
        call("b200pf_tri_mul_noalloc", ptr(z_new), ptr(pm), ptr(w["ln_in_gamma"]), ptr(w["ln_in_beta"]), ptr(w["w_pg_tc"]), ptr(w["w_pout_tc"]),
             ptr(w["w_gout_tc"]), ptr(w["wsum_tc"]), ptr(w["wb_tc"]), n, int(incoming), stream())
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        assert _lib.device_status() == 0
        assert torch.isfinite(z_new).all()
        # same kernels, same inputs: the two paths must agree far inside the bf16 tier (2e-2)
        upd_new, upd_ref = (z_new - z[0].to(dev)), (z_ref - z[0].to(dev))
        rel = float((upd_new - upd_ref).norm() / upd_ref.norm())
        assert rel < 1e-3, (call_no, rel)


def test_noalloc_rejects_sizes_beyond_its_scratch():
    dev = torch.device("cuda:0")
    z = torch.zeros(8, device=dev)
    lib = _lib.load()
    rc = lib.b200pf_tri_mul_noalloc(z.data_ptr(), None, None, None, None, None, None, None, None, 129, 0, None)
    assert rc == -2
    assert "exceeds the built-in scratch" in _lib.last_error()
