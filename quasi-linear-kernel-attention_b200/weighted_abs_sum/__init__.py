"""Drop-in for the reference package `weighted_abs_sum`
(Weighted_Abs_Sum/weighted_abs_sum/__init__.py:1-13)."""

from weighted_abs_sum.ops import (
    weighted_abs_sum,
    weighted_abs_sum_full,
    weighted_sgn_sum,
    weighted_abs_sum_shifted,
    set_keops_cutoff,
)

__all__ = [
    "weighted_abs_sum",
    "weighted_abs_sum_full",
    "weighted_sgn_sum",
    "weighted_abs_sum_shifted",
    "set_keops_cutoff",
]
