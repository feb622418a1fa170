"""Token balancing across data-parallel ranks before a training mini-batch.

Every rank rolls out its own prompts, so the ranks enter the training phase with different numbers of tokens (response
lengths are random) and the optimizer step waits for the fullest rank.  In pure data parallelism any rank can train on
any row, and once the loss reduction has been folded into the advantages (``PPOTrainer._normalize_advantages``) a row
carries everything its loss term needs.  So the rows of a mini-batch are re-dealt: all ranks exchange their row
lengths, compute the same longest-first assignment with an equal number of rows per rank, and move the rows with one
``all_to_all`` per tensor.  The summed gradient is unchanged; only who computes which term changes.

The reference balances inside its dispatcher before the data leaves the driver
(skyrl/backends/skyrl_train/workers/worker_dispatch.py, ``balance_batch`` / sequence-length balanced partitioning);
here there is no driver, so the ranks trade rows among themselves.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .batch import TrainingInputBatch


def plan_assignment(lens_by_rank: Sequence[Sequence[int]]) -> List[List[int]]:
    """``dest[r][i]`` = rank that will train row ``i`` of rank ``r``.  Longest rows first, each to the rank with the
    fewest tokens so far among those that still have room; every rank ends up with as many rows as it started with
    (all ranks hold the same number); between equally loaded candidates the row's own rank wins."""
    W = len(lens_by_rank)
    cap = [len(x) for x in lens_by_rank]
    rows = sorted(((int(l), r, i) for r, ls in enumerate(lens_by_rank) for i, l in enumerate(ls)),
                  key=lambda t: (-t[0], t[1], t[2]))
    load, count = [0] * W, [0] * W
    dest = [[0] * len(x) for x in lens_by_rank]
    for l, r, i in rows:
        best = None
        for d in range(W):
            if count[d] >= cap[d]:
                continue
            key = (load[d], 0 if d == r else 1, d)
            if best is None or key < best[0]:
                best = (key, d)
        d = best[1]
        dest[r][i] = d
        load[d] += l
        count[d] += 1
    return dest


def _pad_to(batch: TrainingInputBatch, keys, S: int, R: int, P_new: int, R_new: int) -> TrainingInputBatch:
    """Widen a batch laid out as [left-padded prompt | response, right-padded] to prompt width ``P_new`` and response
    width ``R_new``: full-width fields grow on both sides, response-width fields on the right, zeros everywhere (the
    attention and loss masks of the new columns are therefore zero)."""
    out = TrainingInputBatch({}, metadata=dict(batch.metadata or {}))
    for k, v in batch.items():
        if v is None or k not in keys or v.dim() < 2:
            out[k] = v
        elif v.shape[1] == S and k in ("sequences", "attention_mask", "position_ids"):
            out[k] = torch.nn.functional.pad(v, (P_new - (S - R), R_new - R))
        elif k == "rollout_expert_indices":  # [B, S, layers, k]: new columns carry no recorded routing
            out[k] = torch.nn.functional.pad(v, (0, 0, 0, 0, P_new - (S - R), R_new - R), value=-1)
        elif k == "router_padding_mask":
            out[k] = torch.nn.functional.pad(v, (P_new - (S - R), R_new - R), value=True)
        elif v.shape[1] == R:
            out[k] = torch.nn.functional.pad(v, (0, R_new - R))
        else:
            out[k] = v
    if "response_length" in out.metadata:
        out.metadata["response_length"] = R_new
    return out


def balance_rows_across_ranks(batch: TrainingInputBatch, rank: int, world: int, group=None
                              ) -> Tuple[TrainingInputBatch, Optional[dict]]:
    """Returns the re-dealt batch and a small report (tokens before / after, rows moved), or the batch unchanged and
    ``None`` when balancing does not apply (one rank, uneven row counts, non-tensor fields)."""
    if world <= 1 or not dist.is_initialized():
        return batch, None
    keys = [k for k, v in batch.items() if v is not None]
    if any(not isinstance(batch[k], torch.Tensor) for k in keys):
        return batch, None
    B = batch.batch_size
    lens = batch["attention_mask"].sum(1).to(torch.int64).cpu()
    gathered = [torch.empty_like(lens) for _ in range(world)]
    sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([B], dtype=torch.int64), group=group)
    if any(int(s) != B for s in sizes):
        return batch, None  # ranks hold different numbers of rows (dynamic sampling leftovers): leave as is
    dist.all_gather(gathered, lens, group=group)
    lens_by_rank = [g.tolist() for g in gathered]
    # every rank pads its batch to its own longest prompt / response: bring all ranks to common widths first
    S, R = int(batch["sequences"].shape[1]), int(batch["response_mask"].shape[1])
    dims = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(dims, torch.tensor([S - R, R], dtype=torch.int64), group=group)
    P_new, R_new = max(int(d[0]) for d in dims), max(int(d[1]) for d in dims)
    if (P_new, R_new) != (S - R, R):
        batch = _pad_to(batch, keys, S, R, P_new, R_new)
    widths = [None] * world
    dist.all_gather_object(widths, {k: tuple(batch[k].shape[1:]) for k in keys}, group=group)
    if any(w != widths[0] for w in widths):
        return batch, None  # a field whose width this module does not understand differs between ranks
    dest = plan_assignment(lens_by_rank)
    mine = torch.tensor(dest[rank], dtype=torch.int64)
    order = torch.argsort(mine, stable=True)                 # my rows grouped by destination
    send_counts = torch.bincount(mine, minlength=world).tolist()
    recv_counts = [sum(1 for d in dest[s] if d == rank) for s in range(world)]
    assert sum(recv_counts) == B
    out = TrainingInputBatch({}, metadata=dict(batch.metadata or {}))
    for k in keys:
        t = batch[k]
        row = t[0].numel() if t.dim() > 1 else 1
        src = t.index_select(0, order.to(t.device)).contiguous().view(-1)
        dst = torch.empty(B * row, dtype=t.dtype, device=t.device)
        dist.all_to_all_single(dst, src, [c * row for c in recv_counts], [c * row for c in send_counts], group=group)
        out[k] = dst.view(B, *t.shape[1:])
    for k, v in batch.items():
        if v is None:
            out[k] = None
    if out.metadata.get("uids") is not None:
        out.metadata["uids"] = None  # rows of a prompt are no longer together; nothing after this point groups by prompt
    before = [sum(x) for x in lens_by_rank]
    after = [0] * world
    moved = 0
    for r in range(world):
        for i, d in enumerate(dest[r]):
            after[d] += lens_by_rank[r][i]
            moved += int(d != r)
    return out, {"max_tokens_before": max(before), "max_tokens_after": max(after), "mean_tokens": sum(before) / world,
                 "rows_moved": moved}
