"""Generate the golden fixtures in this folder from the reference's own CPU Pairformer.

Run where the reference checkout is importable:

    python tests/golden/make_golden.py --reference /path/to/tt-boltz

It imports ``tt_bio.reference`` with ``ttnn`` (the one missing import, a device library) replaced
by a stub, builds ``PairformerModule`` / ``PairformerNoSeqModule`` in eval mode, loads the seeded
weights of ``tt_boltz_b200.synthetic.make_weights`` through ``load_state_dict(strict=True)``
(which also proves the key names and shapes), runs fp32 forward passes on seeded inputs and
stores the outputs.  Weights are NOT stored (12 MB per layer): a fixture carries the generator
arguments plus a checksum of the regenerated weights, and the tests re-derive them.
"""
from __future__ import annotations

import argparse
import os
import sys
from unittest.mock import MagicMock

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tt_boltz_b200 import synthetic  # noqa: E402


def weight_checksum(sd) -> float:
    acc = 0.0
    for i, k in enumerate(sorted(sd)):
        acc += float(sd[k].double().abs().sum()) * (1 + (i % 7))
    return acc


CASES = {
    # name: (N, blocks, with_s, mask kind, affine_jitter, std, taps)
    "layer_n16_taps": dict(n=16, blocks=1, with_s=True, mask="general", jitter=0.3, std=0.05, taps=True),
    "layer_n24_general_mask": dict(n=24, blocks=1, with_s=True, mask="general", jitter=0.3, std=0.05, taps=False),
    "stack2_n20_tailpad": dict(n=20, blocks=2, with_s=True, mask="tail", jitter=0.0, std=0.02, taps=False),
    "noseq2_n18_chain": dict(n=18, blocks=2, with_s=False, mask="chain", jitter=0.2, std=0.05, taps=False),
    "layer_n32_ones": dict(n=32, blocks=1, with_s=True, mask="ones", jitter=0.0, std=0.02, taps=False),
}


def build_masks(kind: str, n: int):
    if kind == "ones":
        return synthetic.tail_padding_mask(n, 0)
    if kind == "tail":
        return synthetic.tail_padding_mask(n, 3)
    if kind == "chain":
        m, pm, _ = synthetic.chain_block_mask(n, 3, n_pad=2, seed=2, keep_inter_chain=False)
        return m, pm
    if kind == "general":
        g = torch.Generator().manual_seed(7)
        m, pm = synthetic.tail_padding_mask(n, 4)
        pm = pm * (torch.rand(1, n, n, generator=g) > 0.2).float()
        return m, pm
    raise ValueError(kind)


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
        sd = synthetic.make_weights(nb, seed=1, std=c["std"], affine_jitter=c["jitter"], with_s=c["with_s"])
        if c["with_s"]:
            mod = PairformerModule(384, 128, nb, v2=True).eval()
        else:
            mod = PairformerNoSeqModule(128, nb).eval()
        ref_keys = [k for k, _ in mod.named_parameters()]
        assert ref_keys == list(sd.keys()), "key order / names differ from the reference"
        mod.load_state_dict(sd, strict=True)
        s, z = synthetic.make_inputs(n, seed=0, with_s=c["with_s"])
        m, pm = build_masks(c["mask"], n)
        out = {"n": n, "blocks": nb, "with_s": c["with_s"], "mask_kind": c["mask"], "jitter": c["jitter"],
               "std": c["std"], "weight_checksum": weight_checksum(sd),
               "mask": m.numpy(), "pair_mask": pm.numpy()}
        if c["with_s"]:
            if c["taps"]:
                L = mod.layers[0]
                zt = z
                zt = zt + L.tri_mul_out(zt, mask=pm, use_kernels=False); out["tap_tri_mul_out"] = zt.numpy()
                zt = zt + L.tri_mul_in(zt, mask=pm, use_kernels=False); out["tap_tri_mul_in"] = zt.numpy()
                zt = zt + L.tri_att_start(zt, mask=pm, chunk_size=None, use_kernels=False); out["tap_tri_att_start"] = zt.numpy()
                zt = zt + L.tri_att_end(zt, mask=pm, chunk_size=None, use_kernels=False); out["tap_tri_att_end"] = zt.numpy()
                zt = zt + L.transition_z(zt); out["tap_transition_z"] = zt.numpy()
            s_out, z_out = mod(s, z, m, pm, use_kernels=False)
            out["s_out"] = s_out.numpy()
        else:
            z_out = mod(z, pm, use_kernels=False)
        out["z_out"] = z_out.numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, "->", path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
