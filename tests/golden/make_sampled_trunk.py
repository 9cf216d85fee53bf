"""Sampled golden fixture of the full-size trunk from the reference's own CPU Pairformer.

    python tests/golden/make_sampled_trunk.py --reference /path/to/tt-boltz [--n 1024 --blocks 64]

Runs ``tt_bio.reference.PairformerModule`` (fp32, eval, use_kernels=False, ``ttnn`` stubbed) on the
benchmark's own inputs: ``synthetic.make_inputs(n, seed=0)``, ``synthetic.make_weights(blocks, seed=1)``,
all-ones masks (or, with ``--pad-frac``, ``synthetic.random_padding_mask``).  One block at N = 1024 takes about half a minute on 8 cores, 64 blocks about 40 minutes,
so the outputs cannot be recomputed per test run; a full z is 512 MiB, so it cannot be committed either.
The fixture therefore keeps, after the block counts in ``--snapshots``:

  * z at 65 536 fixed pseudo-random positions (flat indices into [N, N, 128], seed 5) plus ||z||_2,
  * the whole of s [N, 384].

rel-L2 over the sampled entries estimates the whole-tensor figure to a few percent (65 536 samples of a
quantity with no structure in the sampling pattern).  Weights are re-derived from the seed by the tests; a
checksum guards against generator drift.
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from unittest.mock import MagicMock

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tt_boltz_b200 import synthetic  # noqa: E402
from tests.golden.make_golden import weight_checksum  # noqa: E402

N_SAMPLES = 65536


def sample_index(n: int, c: int = 128, seed: int = 5) -> torch.Tensor:
    """Fixed flat positions into z [n, n, c] (sorted, distinct draws not required)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.sort(torch.randint(0, n * n * c, (N_SAMPLES,), generator=g)).values


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--n", type=int, default=1024)
    ap.add_argument("--blocks", type=int, default=64)
    ap.add_argument("--snapshots", default="1,8,64")
    ap.add_argument("--threads", type=int, default=os.cpu_count() or 1)
    ap.add_argument("--pad-frac", type=float, default=0.0,
                    help="fraction of tokens masked at random (seed 3); 0 = all-ones masks")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.modules["ttnn"] = MagicMock(name="ttnn")
    torch.set_grad_enabled(False)
    torch.set_num_threads(args.threads)
    torch.set_float32_matmul_precision("highest")
    from tt_bio.reference import PairformerModule

    n, nb = args.n, args.blocks
    snaps = sorted(int(x) for x in args.snapshots.split(",") if int(x) <= nb)
    sd = synthetic.make_weights(nb, seed=1)
    mod = PairformerModule(384, 128, nb, v2=True).eval()
    assert [k for k, _ in mod.named_parameters()] == list(sd.keys())
    mod.load_state_dict(sd, strict=True)
    s, z = synthetic.make_inputs(n, seed=0)
    m, pm = (synthetic.random_padding_mask(n, args.pad_frac, seed=3) if args.pad_frac > 0
             else synthetic.tail_padding_mask(n, 0))
    idx = sample_index(n)
    out = {"n": n, "blocks": nb, "pad_frac": args.pad_frac, "mask": m[0].numpy(), "snapshots": np.array(snaps), "index": idx.numpy(), "weight_checksum": weight_checksum(sd),
           "z_in_samples": z.reshape(-1)[idx].numpy()}
    t0 = time.time()

    def hook_for(block: int):
        def hook(_mod, _inp, result):
            s_b, z_b = result
            print(f"block {block}: {time.time() - t0:.0f} s, rms z {float(z_b.pow(2).mean().sqrt()):.4f}", flush=True)
            if block in snaps:
                out[f"z_samples_{block}"] = z_b.reshape(-1)[idx].numpy().copy()
                out[f"z_norm_{block}"] = float(z_b.double().norm())
                out[f"s_{block}"] = s_b[0].numpy().copy()
        return hook

    for i, layer in enumerate(mod.layers):
        layer.register_forward_hook(hook_for(i + 1))
    mod(s, z, m, pm, use_kernels=False)
    path = args.out or os.path.join(HERE, "sampled", f"trunk_n{n}_b{nb}{'_pad' if args.pad_frac > 0 else ''}.npz")
    os.makedirs(os.path.dirname(path), exist_ok=True)
    np.savez_compressed(path, **out)
    print("->", path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
