"""Partition of the hard path over the GPUs of one node.

Every (batch, head) is an independent problem (the reference's task tables enumerate them one by
one, dism_v3/src/host/hard_summary.cpp:28,44-48), so ranks take contiguous slices of heads and no
collective touches the data path; dtau is per head and needs no reduction either.
"""


def head_range(heads, rank, world):
    """Contiguous [lo, hi) of heads for `rank`; sizes differ by at most one."""
    base, extra = divmod(heads, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


_HEAD_AXIS = dict(sq=2, sk=2, v=2, dout=2, q=2, k=2, out=2, iq=1, ik=1, hard=1, lse2=1, tau=0, eq=0, ek=0)


def shard_operands(operands, rank, world):
    """Slice every operand (numpy arrays or torch tensors, keyed by the names above) to this rank's heads."""
    heads = operands['tau'].shape[0]
    lo, hi = head_range(heads, rank, world)
    out = {}
    for name, value in operands.items():
        axis = _HEAD_AXIS[name]
        index = [slice(None)] * value.ndim
        index[axis] = slice(lo, hi)
        piece = value[tuple(index)]
        out[name] = piece.contiguous() if hasattr(piece, 'contiguous') else piece.copy()
    return out
