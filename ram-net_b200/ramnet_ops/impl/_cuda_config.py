"""Index capacities of the CUDA backend (mirrors packages/ramnet-ops/src/ramnet_ops/impl/_cuda_config.py).

Slot indices are int32, so one call may address at most 2^31 slots (B*H*A).  Unlike the
reference, element offsets into the slot state are 64-bit inside the kernels, so the state
itself (B*H*A*C elements) is NOT limited to 2^31."""
from ramnet_ops import _C

INT_BITS = _C.INT_BITS
INT_MAX = (1 << (INT_BITS - 1)) - 1
# one magnitude bit is kept free for intermediate address arithmetic
ADDRESS_LIMIT = 1 << (INT_BITS - 2)


def check_int_capacity(*sizes: int) -> None:
    assert all(0 <= size < INT_MAX for size in sizes), f"CUDA index overflow: sizes={sizes}, limit={INT_MAX}."
