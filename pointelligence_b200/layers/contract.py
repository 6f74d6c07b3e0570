"""Structural facts about a triplet index, fixed when it is built (mirror of
``layers/contract.py:27-64``)."""
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class TripletContract:
    """``k_sorted``: triplets ascend by tap.  ``exact_cover_out`` / ``exact_cover_in``:
    every output / input row occurs in exactly one triplet.  ``uniform_seg_len``:
    every tap owns exactly this many triplets (None = ragged)."""
    k_sorted: bool = True
    exact_cover_out: bool = False
    exact_cover_in: bool = False
    uniform_seg_len: Optional[int] = None

    @classmethod
    def submanifold(cls) -> "TripletContract":
        return cls()
