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
    from oracle import pairformer_oracle as orc
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    sd = _strip(synthetic.make_weights(1, seed=5, std=0.05, affine_jitter=0.3, with_s=False))
    for call_no, (n, incoming, seed) in enumerate([(100, False, 4), (72, True, 6)]):
        _, z = synthetic.make_inputs(n, seed=seed, with_s=False)
        g = torch.Generator().manual_seed(seed)
        pm_cpu = (torch.rand(n, n, generator=g) > 0.2).float()
        pm = pm_cpu.to(torch.uint8).to(dev)
        pre = "tri_mul_in." if incoming else "tri_mul_out."
        w = weights.pack_trimul(sd, pre, dev)
        z_ref = z[0].to(dev).clone()
        ops.tri_mul_bf16(z_ref, pm, w, ops.Workspace(n, dev), incoming)
        z_new = z[0].to(dev).clone()
        args = (ptr(z_new), ptr(pm), ptr(w["ln_in_gamma"]), ptr(w["ln_in_beta"]), ptr(w["w_pg_tc"]), ptr(w["w_pout_tc"]),
                ptr(w["w_gout_tc"]), ptr(w["wsum_tc"]), ptr(w["wb_tc"]), n, int(incoming), stream())
        if call_no == 0:
            # warm-up on a copy: loads the kernels and looks up the array's address, the only things a first
            # call may do that touch device memory behind the caller's back
            z_warm = z[0].to(dev).clone()
            call("b200pf_tri_mul_noalloc", ptr(z_warm), *args[1:])
            torch.cuda.synchronize()
        # the driver's own count of free device memory (torch's allocator statistics would not see a
        # cudaMalloc made inside the library)
        free_before = torch.cuda.mem_get_info(dev)[0]
        call("b200pf_tri_mul_noalloc", *args)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before, "device memory was allocated during the call"
        assert _lib.device_status() == 0
        assert torch.isfinite(z_new).all()
        # the same three kernels on the same inputs, only the planes live elsewhere: bit for bit
        assert torch.equal(z_new, z_ref), (call_no, float((z_new - z_ref).abs().max()))
        # and against the CPU oracle, inside the bf16 tier
        with torch.no_grad():
            upd = orc.tri_mul(z[0], sd, pre[:-1], pm_cpu, incoming)
        rel = float((z_new.cpu() - z[0] - upd).norm() / upd.norm())
        assert rel < 2e-2, (call_no, rel)


def test_noalloc_sources_name_no_allocating_call():
    """CPU-side guard: neither the entry point nor the three stage wrappers it calls may name an allocating or
    freeing runtime routine."""
    import os
    import re
    csrc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tt_boltz_b200", "csrc")
    bad = re.compile(r"cudaMalloc|cudaFree|cudaMemPool|cuMemAlloc|cuMemFree|cudaHostAlloc|at::empty|torch::")
    for name in ("trimul_noalloc.cu", "row512_tc.cu", "trimul_gemm.cu", "trimul_epilogue_tc.cu", "tmap.cuh", "common.cuh"):
        text = open(os.path.join(csrc, name)).read()
        assert not bad.search(text), name


def test_noalloc_rejects_sizes_beyond_its_scratch():
    dev = torch.device("cuda:0")
    z = torch.zeros(8, device=dev)
    lib = _lib.load()
    rc = lib.b200pf_tri_mul_noalloc(z.data_ptr(), None, None, None, None, None, None, None, None, 129, 0, None)
    assert rc == -2
    assert "exceeds the built-in scratch" in _lib.last_error()
