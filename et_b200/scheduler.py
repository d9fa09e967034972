"""Length-bucketed batching for serving-style variable-length requests: the caller's side of the packed
variable-length path (`Encoder_length` of the reference runs one sequence per object, encoder/encoder.cu:116-149).

Requests are grouped so that (a) a batch never exceeds a token budget (scratch and latency are bounded), (b) the
sequences of a batch have similar lengths, which keeps the 128-query attention blocks full and lets repeated
length patterns hit the layer's graph-replay cache, and (c) the original order is recoverable. Pure host logic."""
from dataclasses import dataclass
from typing import List, Sequence


@dataclass
class Batch:
    indices: List[int]    # request indices, ascending
    lengths: List[int]    # their lengths, same order
    padded_to: int        # bucket ceiling: every length <= padded_to

    @property
    def tokens(self) -> int:
        return sum(self.lengths)


def bucket_ceiling(length: int, width: int) -> int:
    """Smallest multiple of `width` that holds `length` (at least one bucket)."""
    if width <= 0:
        raise ValueError("bucket width must be positive")
    return max(width, (length + width - 1) // width * width)


def bucket_by_length(lengths: Sequence[int], max_tokens: int, width: int = 64, max_batch: int = 0) -> List[Batch]:
    """Groups requests by bucket ceiling, then cuts each group into batches of at most `max_tokens` packed tokens
    (and `max_batch` sequences, if given). Batches come out in ascending bucket order; inside a batch the request
    indices ascend. A request longer than `max_tokens` gets a batch of its own."""
    if max_tokens <= 0:
        raise ValueError("max_tokens must be positive")
    if any(l < 0 for l in lengths):
        raise ValueError("negative length")
    groups = {}
    for i, l in enumerate(lengths):
        if l == 0:
            continue   # nothing to compute; restore_order leaves its slot empty
        groups.setdefault(bucket_ceiling(l, width), []).append(i)
    out: List[Batch] = []
    for ceil in sorted(groups):
        cur: List[int] = []
        tok = 0
        for i in groups[ceil]:
            l = lengths[i]
            if cur and (tok + l > max_tokens or (max_batch and len(cur) >= max_batch)):
                out.append(Batch(cur, [lengths[j] for j in cur], ceil))
                cur, tok = [], 0
            cur.append(i)
            tok += l
        if cur:
            out.append(Batch(cur, [lengths[j] for j in cur], ceil))
    return out


def padding_waste(batches: Sequence[Batch]) -> float:
    """Fraction of attention-block work spent on padding if every sequence were padded to its bucket ceiling."""
    real = sum(sum(b.lengths) for b in batches)
    padded = sum(b.padded_to * len(b.lengths) for b in batches)
    return 0.0 if padded == 0 else 1.0 - real / padded


def restore_order(batches: Sequence[Batch], outputs: Sequence[Sequence], n_requests: int) -> List:
    """outputs[b][k] is the result for request batches[b].indices[k]; returns them in request order (None for
    zero-length requests)."""
    res = [None] * n_requests
    for b, outs in zip(batches, outputs):
        if len(outs) != len(b.indices):
            raise ValueError("one output per request of the batch is required")
        for i, o in zip(b.indices, outs):
            res[i] = o
    return res
