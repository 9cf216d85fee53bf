"""Generate the fixtures in this folder: the reference's own CPU Pairformer at the widths of its other call sites.

Run where the reference checkout is importable:

    python tests/golden/widths/make_widths.py --reference /path/to/tt-boltz

Same recipe as ``tests/golden/make_golden.py`` (``tt_bio.reference`` imported with ``ttnn`` stubbed, seeded weights of
``tt_boltz_b200.synthetic.make_weights`` loaded with ``strict=True``, fp32 forward in eval mode, outputs stored, weights
re-derived by the tests from the stored generator arguments and checked by a checksum), for

* the template stack: ``PairformerNoSeqModule(64, 2)`` with four triangle heads of width 32 (tt_bio/boltz2.py:3749-3760),
* a block with pair width 256 and eight triangle heads, with the single track (the Protenix-v2 dimensions,
  tt_bio/protenix.py:939-953, on the reference's Boltz-2 modules, which its Protenix port maps onto).
"""
from __future__ import annotations

import argparse
import os
import sys
from unittest.mock import MagicMock

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(HERE))))

from tests.golden.make_golden import build_masks, weight_checksum  # noqa: E402
from tt_boltz_b200 import synthetic  # noqa: E402

CASES = {
    "template_noseq2_c64_n20_chain": dict(n=20, blocks=2, with_s=False, mask="chain", jitter=0.2, std=0.05, c_z=64, tri_heads=4),
    "layer_c256_h8_n12_general": dict(n=12, blocks=1, with_s=True, mask="general", jitter=0.2, std=0.03, c_z=256, tri_heads=8),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of moritztng/tt-boltz (the directory that holds tt_bio/)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.modules["ttnn"] = MagicMock(name="ttnn")
    torch.set_grad_enabled(False)
    torch.set_float32_matmul_precision("highest")
    from tt_bio.reference import PairformerModule, PairformerNoSeqModule

    for name, c in CASES.items():
        n, nb = c["n"], c["blocks"]
        sd = synthetic.make_weights(nb, seed=1, std=c["std"], affine_jitter=c["jitter"], with_s=c["with_s"], c_z=c["c_z"],
                                    tri_heads=c["tri_heads"])
        if c["with_s"]:
            mod = PairformerModule(384, c["c_z"], nb, pairwise_num_heads=c["tri_heads"], v2=True).eval()
        else:
            mod = PairformerNoSeqModule(c["c_z"], nb, pairwise_num_heads=c["tri_heads"]).eval()
        assert [k for k, _ in mod.named_parameters()] == list(sd.keys()), "key order / names differ from the reference"
        mod.load_state_dict(sd, strict=True)
        s, z = synthetic.make_inputs(n, c_z=c["c_z"], seed=0, with_s=c["with_s"])
        m, pm = build_masks(c["mask"], n)
        out = {"n": n, "blocks": nb, "with_s": c["with_s"], "mask_kind": c["mask"], "jitter": c["jitter"], "std": c["std"],
               "c_z": c["c_z"], "tri_heads": c["tri_heads"], "weight_checksum": weight_checksum(sd),
               "mask": m.numpy(), "pair_mask": pm.numpy()}
        if c["with_s"]:
            s_out, z_out = mod(s, z, m, pm, use_kernels=False)
            out["s_out"] = s_out.numpy()
        else:
            z_out = mod(z, pm, use_kernels=False)
        out["z_out"] = z_out.numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, "->", os.path.getsize(path) // 1024, "KiB", float(z_out.abs().mean()))


if __name__ == "__main__":
    main()
