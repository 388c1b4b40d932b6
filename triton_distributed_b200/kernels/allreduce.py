"""AllReduce method enumeration (API parity with ``python/triton_dist/kernels/allreduce.py:28-61``)."""
from __future__ import annotations

import enum


class AllReduceMethod(enum.Enum):
    Unknown = 0
    DoubleTree = 1
    OneShot = 2
    TwoShot = 3
    OneShot_TMA = 4
    OneShot_Multimem = 5
    TwoShot_Multimem = 6
    TwoShot_Multimem_ST = 7


_STR_TO_METHOD = {
    "double_tree": AllReduceMethod.DoubleTree,
    "one_shot": AllReduceMethod.OneShot,
    "two_shot": AllReduceMethod.TwoShot,
    "one_shot_tma": AllReduceMethod.OneShot_TMA,
    "one_shot_multimem": AllReduceMethod.OneShot_Multimem,
    "two_shot_multimem": AllReduceMethod.TwoShot_Multimem,
    "two_shot_multimem_st": AllReduceMethod.TwoShot_Multimem_ST,
}


def to_allreduce_method(name: str) -> AllReduceMethod:
    try:
        return _STR_TO_METHOD[name]
    except KeyError:
        raise ValueError(f"unknown allreduce method {name!r}; choose from {sorted(_STR_TO_METHOD)}") from None


def get_allreduce_methods() -> list[str]:
    return list(_STR_TO_METHOD)
