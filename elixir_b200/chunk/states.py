"""Life cycle of a tensor stored in a chunk (counterpart of ``elixir/chunk/core/states.py``).

free -> hold -> compute -> hold -> compute -> hold_after_bwd -> ready_for_reduce -> hold
"""
from enum import Enum


class TensorState(Enum):
    FREE = 0
    COMPUTE = 1
    HOLD = 2
    HOLD_AFTER_BWD = 3
    READY_FOR_REDUCE = 4


_NEXT = {
    TensorState.FREE: {TensorState.HOLD, TensorState.COMPUTE},
    TensorState.HOLD: {TensorState.FREE, TensorState.COMPUTE},
    TensorState.COMPUTE: {TensorState.HOLD, TensorState.HOLD_AFTER_BWD},
    TensorState.HOLD_AFTER_BWD: {TensorState.COMPUTE, TensorState.READY_FOR_REDUCE},
    TensorState.READY_FOR_REDUCE: {TensorState.HOLD},
}

legal_ts_update_list = [(old, new) for old, news in _NEXT.items() for new in sorted(news, key=lambda s: s.value)]


def ts_update_sanity_check(old_state: TensorState, new_state: TensorState) -> bool:
    if new_state not in _NEXT[old_state]:
        raise RuntimeError(f'illegal tensor state updating: {old_state} -> {new_state}')
    return True
