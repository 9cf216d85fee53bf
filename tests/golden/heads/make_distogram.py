"""Generate ``distogram_n12.npz`` from the reference's own ``DistogramModule`` (tt_bio/boltz2.py:2334-2368).

    python tests/golden/heads/make_distogram.py --reference /path/to/tt-boltz

``tt_bio.boltz2`` is imported with ``ttnn`` (a device library, its one missing import) replaced by a stub; the module
gets seeded weights and a seeded, NON-symmetric pair tensor (the head symmetrises it).  Stored: the module's state
dict under its own key names, z and the output.
"""
from __future__ import annotations

import argparse
import os
import sys
from unittest.mock import MagicMock

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a tt-boltz checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.modules.setdefault("ttnn", MagicMock(name="ttnn"))
    from tt_bio.boltz2 import DistogramModule

    torch.set_grad_enabled(False)
    n, c, bins = 12, 128, 64
    g = torch.Generator().manual_seed(31)
    mod = DistogramModule(c, bins).eval()
    w = {"distogram.weight": torch.randn(bins, c, generator=g) / c ** 0.5, "distogram.bias": 0.3 * torch.randn(bins, generator=g)}
    mod.load_state_dict(w, strict=True)
    z = torch.randn(1, n, n, c, generator=g)
    out = mod(z)
    np.savez_compressed(os.path.join(HERE, "distogram_n12.npz"), z=z.numpy(), out=out.numpy().astype(np.float32),
                        **{"w::" + k: v.numpy() for k, v in w.items()})
    print(tuple(out.shape), float(out.abs().mean()))


if __name__ == "__main__":
    main()
