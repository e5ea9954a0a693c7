"""Spreading independent work over the GPUs of one box.

The quantized path shards by rows: every activation row (token) of a linear,
every sequence of an encoder batch is independent, so ranks take disjoint
slices, weights are replicated and no collective runs on the data path.  The
reference has no such layer: its runtime is one context per (device, stream)
and multi-GPU means independent replicas
(pytorch_blade/pytorch_blade/compiler/mlir/runtime/ral_context.cpp:243-271).
"""
from typing import List, Sequence, Tuple


def row_range(total_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [begin, end) slice of ``total_rows`` for ``rank``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(total_rows, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def balance_sequences(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Assigns sequence indices to ranks so that padded work is even.

    A rank pads its sequences to its own longest one, so its cost is
    ``count * max_len``.  Sequences are sorted by length (longest first) and cut
    into at most ``world`` contiguous runs, which keeps similar lengths together;
    the smallest bound B for which greedy filling (``count * max_len <= B``)
    needs no more than ``world`` runs is found by bisection, and that filling is
    returned.  Ranks beyond the number of runs get nothing.
    """
    n = len(lengths)
    if world <= 0:
        raise ValueError("world must be positive")
    order = sorted(range(n), key=lambda i: (-lengths[i], i))
    out: List[List[int]] = [[] for _ in range(world)]
    if n == 0:
        return out

    def fill(bound: int) -> List[List[int]]:
        runs: List[List[int]] = []
        pos = 0
        while pos < n:
            max_len = max(lengths[order[pos]], 1)
            take = max(1, bound // max_len)
            runs.append(order[pos:pos + take])
            pos += take
        return runs

    lo, hi = max(lengths[order[0]], 1), max(lengths[order[0]], 1) * n
    while lo < hi:
        mid = (lo + hi) // 2
        if len(fill(mid)) <= world:
            hi = mid
        else:
            lo = mid + 1
    runs = fill(lo)
    # Idle ranks help nobody: while some rank would get nothing, halve the most expensive
    # run that can still be cut (this never raises the maximum).
    while len(runs) < min(world, n):
        k = max((i for i in range(len(runs)) if len(runs[i]) > 1),
                key=lambda i: len(runs[i]) * lengths[runs[i][0]])
        run = runs[k]
        half = len(run) // 2
        runs[k:k + 1] = [run[:half], run[half:]]
    for r, run in enumerate(runs):
        out[r] = sorted(run)
    return out


def packed_cost(length: int) -> float:
    """Relative cost of one sequence when the batch is packed (no padding rows): the linears, norms and
    quantizes grow with the tokens, self-attention with their square (its share is about a tenth at 512
    tokens of a BERT-base layer, more in time than in operations)."""
    return length * (1.0 + length / 1500.0)


def balance_packed(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Assigns sequence indices to ranks so that the packed work (``packed_cost``) is even: longest
    first, each sequence to the rank with the least work so far.  Every rank gets a sequence while
    there are any left; ties go to the lower rank, so the result is the same on every rank."""
    if world <= 0:
        raise ValueError("world must be positive")
    out: List[List[int]] = [[] for _ in range(world)]
    load = [0.0] * world
    for i in sorted(range(len(lengths)), key=lambda i: (-lengths[i], i)):
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += packed_cost(max(int(lengths[i]), 1))
    return [sorted(a) for a in out]


def padded_cost(lengths: Sequence[int], assignment: Sequence[Sequence[int]]) -> List[int]:
    """Rows each rank processes when it pads to its own longest sequence."""
    return [len(a) * max((lengths[i] for i in a), default=0) for a in assignment]


def column_range(total_cols: int, world: int, rank: int, multiple: int = 128) -> Tuple[int, int]:
    """Slice of output channels for a column-parallel (N-split) linear; slice
    boundaries fall on ``multiple`` so that every rank's tile grid is full."""
    blocks = (total_cols + multiple - 1) // multiple
    b0, b1 = row_range(blocks, world, rank)
    return min(b0 * multiple, total_cols), min(b1 * multiple, total_cols)
