"""How the decode path is spread over the GPUs of one box (one process per GPU).

Two ways, both without any reference counterpart (the reference is single-device):

* by sequence — sequences are independent, each rank owns the pages, tables and a weight replica
  for its share of the batch; no collective touches the attention path;
* by KV range — one very long sequence is cut into contiguous page-aligned token ranges; every
  rank computes the partial softmax state (m, l, acc[512]) of its range for the replicated query,
  the states are exchanged with ONE all-gather and merged locally by log-sum-exp, followed by the
  W_UV projection.  The token appended in a step goes to the rank that owns the tail.
"""
from __future__ import annotations

import numpy as np

PART = 514   # floats per head of a partial state: m (log2 domain), l, acc[512]


def shard_batch(n_seq: int, world: int, rank: int) -> range:
    """Contiguous, near-equal share of a uniform batch."""
    base, extra = divmod(n_seq, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_by_load(lengths, world: int) -> list[list[int]]:
    """Ragged batch: greedy longest-first assignment that balances the cache bytes per rank."""
    order = sorted(range(len(lengths)), key=lambda i: -int(lengths[i]))
    loads = [0] * world
    out = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (loads[k], k))
        out[r].append(i)
        loads[r] += int(lengths[i])
    return [sorted(x) for x in out]


def kv_range_slices(seq_len: int, world: int, page_tokens: int = 64) -> list[tuple[int, int]]:
    """Page-aligned [begin, end) token ranges, one per rank; the last rank owns the tail."""
    pages = (seq_len + page_tokens - 1) // page_tokens
    cuts = [min(seq_len, (pages * r // world) * page_tokens) for r in range(world)] + [seq_len]
    return [(cuts[r], cuts[r + 1]) for r in range(world)]


def merge_partials_reference(parts: np.ndarray) -> np.ndarray:
    """float64 log-sum-exp merge of partial states [n_parts][rows][H][514] -> normalised
    o_c [rows][H][512]; mirrors what mla_merge_partials computes before W_UV (used by tests)."""
    p = parts.astype(np.float64)
    m = p[..., 0]
    big = m.max(axis=0)
    w = np.where(np.isfinite(m), np.exp2(m - np.where(np.isfinite(big), big, 0.0)), 0.0)
    l = (w * p[..., 1]).sum(axis=0)
    acc = (w[..., None] * p[..., 2:]).sum(axis=0)
    return acc / np.where(l > 0, l, 1.0)[..., None]


def kv_range_attend(ctx, layer: int, q, partial, gathered, out, group=None) -> None:
    """One layer of a KV-range-sharded step on this rank: partial state of the local range ->
    all-gather over the group (NCCL on GPUs) -> local merge + W_UV.
    partial: float32 [rows][H][514]; gathered: float32 [world][rows][H][514]."""
    import torch.distributed as dist
    ctx.step_attend_partial(layer, q, partial)
    # concatenation form (world*rows leading dimension): accepted by NCCL and gloo alike
    dist.all_gather_into_tensor(gathered.view(-1, *partial.shape[1:]), partial, group=group)
    ctx.merge_partials(layer, gathered.shape[0], partial.shape[0], gathered, out)
