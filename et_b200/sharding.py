"""Batch sharding for multi-GPU runs: sequences are independent, so a batch is split across ranks with no
collective inside the layer loop; only the outputs are gathered. Pure host logic (no CUDA)."""
from typing import List, Sequence, Tuple


def sequence_cost(length: int, d_model: int = 768, d_ff: int = 3072) -> float:
    """Work of one encoder layer on a sequence: linear terms per token plus the L^2 attention term."""
    return length * (8.0 * d_model * d_model + 4.0 * d_model * d_ff) + 4.0 * length * length * d_model


def shard_sequences(seq_lens: Sequence[int], world_size: int, d_model: int = 768,
                    d_ff: int = 3072) -> List[List[int]]:
    """Assigns sequence indices to ranks. Equal lengths: contiguous equal shards (remainder to the first
    ranks). Unequal lengths: longest-processing-time greedy on the per-sequence cost; each rank's list is kept
    in ascending index order so the original order is recoverable."""
    n = len(seq_lens)
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    if n == 0:
        return [[] for _ in range(world_size)]
    if len(set(seq_lens)) == 1:
        base, extra = divmod(n, world_size)
        out, start = [], 0
        for r in range(world_size):
            cnt = base + (1 if r < extra else 0)
            out.append(list(range(start, start + cnt)))
            start += cnt
        return out
    order = sorted(range(n), key=lambda i: (-sequence_cost(seq_lens[i], d_model, d_ff), i))
    loads = [0.0] * world_size
    out = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (loads[k], k))
        out[r].append(i)
        loads[r] += sequence_cost(seq_lens[i], d_model, d_ff)
    return [sorted(s) for s in out]


def token_ranges(seq_lens: Sequence[int]) -> List[Tuple[int, int]]:
    """(first token, one past last token) of each sequence in the packed layout."""
    out, start = [], 0
    for l in seq_lens:
        out.append((start, start + l))
        start += l
    return out


def gather_plan(seq_lens: Sequence[int], shards: List[List[int]]) -> Tuple[int, List[List[Tuple[int, int, int]]]]:
    """For an all-gather of equally sized (padded) per-rank token buffers: returns the padded shard size in
    tokens and, per rank, the list of (offset in the rank's buffer, destination token offset, length) that
    scatters the gathered rows back into the original packed order."""
    ranges = token_ranges(seq_lens)
    sizes = [sum(seq_lens[i] for i in s) for s in shards]
    pad = max(sizes) if sizes else 0
    plan = []
    for s in shards:
        off, moves = 0, []
        for i in s:
            a, b = ranges[i]
            moves.append((off, a, b - a))
            off += b - a
        plan.append(moves)
    return pad, plan
