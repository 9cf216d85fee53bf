"""The reference's own CPU Pairformer modules, imported from the install that oracle/build_ref.py makes.

Test infrastructure (the checker and the timed CPU baseline), never part of the product path.
"""
from __future__ import annotations

import os
import sys
from unittest.mock import MagicMock

_REF = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def available() -> bool:
    return os.path.isfile(os.path.join(_REF, "tt_bio", "reference.py"))


def load():
    """(PairformerModule, PairformerNoSeqModule) of tt_bio/reference.py:918-1139, with the absent ``ttnn`` device
    library replaced by a stub (its module-level uses are a core-grid constant, annotations and an atexit hook)."""
    if not available():
        raise RuntimeError("oracle/_ref is missing: run `python oracle/build_ref.py --reference <tt-boltz checkout>`")
    if _REF not in sys.path:
        sys.path.insert(0, _REF)
    sys.modules.setdefault("ttnn", MagicMock(name="ttnn"))
    from tt_bio.reference import PairformerModule, PairformerNoSeqModule
    return PairformerModule, PairformerNoSeqModule
