"""Tensorisation of rollouts and the packed-token view used by the model.

``convert_prompts_responses_to_batch_tensors`` produces the public padded layout
(reference: skyrl/train/dataset/preprocess.py:90-283): ``sequences [B, max(p_i + r_i)]`` left-padded,
response-level tensors ``[B, max r_i]`` right-aligned.  ``pack_batch`` converts a slice of that
layout into the token-packed form (ids, positions, cu_seqlens) plus the gather/scatter indices that
map per-token log-probabilities back to the right-aligned response grid; the model itself never
sees padding.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


def convert_prompts_responses_to_batch_tensors(
    pad_token_id: int, prompts: Sequence[Sequence[int]], responses: Sequence[Sequence[int]],
    rewards: Sequence[Sequence[float]], loss_masks: Sequence[Sequence[int]],
    logprobs: Optional[Sequence[Sequence[float]]] = None, max_seq_len: Optional[int] = None,
):  # fmt: skip
    """Returns ``(sequences, attention_mask, response_mask, rewards, loss_mask, rollout_logprobs)``."""
    assert len(prompts) == len(responses) and len(prompts) > 0, "need matching, non-empty prompts and responses"
    B = len(prompts)
    lens = [len(p) + len(r) for p, r in zip(prompts, responses)]
    S = max(lens)
    R = max(1, max(len(r) for r in responses))
    seq = torch.full((B, S), pad_token_id, dtype=torch.long)
    att = torch.zeros((B, S), dtype=torch.long)
    rmask = torch.zeros((B, R), dtype=torch.long)
    lmask = torch.zeros((B, R), dtype=torch.float32)
    rew = torch.zeros((B, R), dtype=torch.float32)
    lps = torch.zeros((B, R), dtype=torch.float32) if logprobs is not None else None
    for i, (p, r) in enumerate(zip(prompts, responses)):
        L, n = lens[i], len(r)
        seq[i, S - L:] = torch.tensor(list(p) + list(r), dtype=torch.long)
        att[i, S - L:] = 1
        if n == 0:
            continue
        rmask[i, R - n:] = 1
        assert len(loss_masks[i]) == n, f"loss mask length {len(loss_masks[i])} != response length {n}"
        lmask[i, R - n:] = torch.tensor(loss_masks[i], dtype=torch.float32)
        assert len(rewards[i]) == n, f"per-token reward length {len(rewards[i])} != response length {n}"
        rew[i, R - n:] = torch.tensor(rewards[i], dtype=torch.float32)
        if lps is not None:
            assert len(logprobs[i]) == n
            lps[i, R - n:] = torch.tensor(logprobs[i], dtype=torch.float32)
    if max_seq_len is not None and S > max_seq_len:
        import warnings

        warnings.warn(f"sequence length {S} exceeds max_seq_len {max_seq_len}")
    return seq, att, rmask, rew, lmask, lps


def compute_prompt_boundaries(uids: Sequence[str]) -> List[Tuple[int, int]]:
    """Consecutive runs of equal uid -> [(start, end)] (reference: preprocess.py:286-313)."""
    out: List[Tuple[int, int]] = []
    start = 0
    for i in range(1, len(uids) + 1):
        if i == len(uids) or uids[i] != uids[start]:
            out.append((start, i))
            start = i
    return out


def compute_prompt_mini_batch_boundaries(uids: Sequence[str], prompts_per_mini_batch: int) -> List[Tuple[int, int]]:
    """Mini-batch row ranges that contain ``prompts_per_mini_batch`` whole prompts each."""
    groups = compute_prompt_boundaries(uids)
    out = []
    for g in range(0, len(groups), prompts_per_mini_batch):
        chunk = groups[g : g + prompts_per_mini_batch]
        out.append((chunk[0][0], chunk[-1][1]))
    return out


@dataclass
class PackedView:
    ids: torch.Tensor  # [T] int32 token ids (all real tokens of the rows, concatenated)
    positions: torch.Tensor  # [T] int32 position of each token inside its sequence
    cu_seqlens: torch.Tensor  # [n_rows + 1] int32
    max_seqlen: int
    pred_index: torch.Tensor  # [N] long: packed index of the hidden state that predicts response token k
    targets: torch.Tensor  # [N] int32: the response tokens themselves
    grid_row: torch.Tensor  # [N] long: row in the [n_rows, R] grid
    grid_col: torch.Tensor  # [N] long: column in the right-aligned [n_rows, R] grid
    n_rows: int
    num_actions: int
    total_tokens: int
    routing: Optional[torch.Tensor] = None  # [T, layers, top_k] rollout-time expert ids to replay (-1: none recorded)

    def scatter_to_grid(self, flat: torch.Tensor, fill: float = 0.0) -> torch.Tensor:
        """Place per-response-token values into the right-aligned ``[n_rows, R]`` grid."""
        grid = flat.new_full((self.n_rows, self.num_actions), fill)
        return grid.index_put((self.grid_row, self.grid_col), flat)

    def gather_from_grid(self, grid: torch.Tensor) -> torch.Tensor:
        return grid[self.grid_row, self.grid_col]


def pack_batch(sequences: torch.Tensor, attention_mask: torch.Tensor, response_mask: torch.Tensor, device,
               pad_multiple: int = 0, pad_to: int = 0) -> PackedView:
    """Build the packed view of left-padded ``sequences`` (host-side index arithmetic, one H2D per tensor).

    ``pad_multiple`` > 0 appends one dummy sequence so that the packed length is a multiple of it: activations then
    come in a few repeating sizes, which keeps the caching allocator from growing and flushing its pool step after
    step (the dummy tokens predict nothing and receive no gradient).  ``pad_to`` > 0: a batch that fills at least
    ``pad_to - 2 * pad_multiple`` tokens is padded to exactly ``pad_to`` (bins packed to a token budget)."""
    seq = sequences.cpu()
    att = attention_mask.cpu().bool()
    B, S = seq.shape
    R = response_mask.shape[1]
    lens = att.sum(1)
    rlens = response_mask.cpu().sum(1)
    ids = seq[att].to(torch.int32)
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = lens.cumsum(0)
    pos = torch.cat([torch.arange(int(n), dtype=torch.int32) for n in lens.tolist()]) if B else ids.new_zeros(0)
    rows, cols, pred = [], [], []
    for b in range(B):
        L, n = int(lens[b]), int(rlens[b])
        if n == 0:
            continue
        start = int(cu[b])
        k = torch.arange(n)
        rows.append(torch.full((n,), b, dtype=torch.long))
        cols.append(R - n + k)
        pred.append(start + L - n - 1 + k)  # hidden state at the token before response token k
    if rows:
        grid_row, grid_col, pred_index = torch.cat(rows), torch.cat(cols), torch.cat(pred)
    else:
        grid_row = grid_col = pred_index = torch.zeros(0, dtype=torch.long)
    targets = ids[(pred_index + 1)] if pred_index.numel() else ids.new_zeros(0)
    n_real = int(ids.numel())
    n_pad = 0
    if pad_to and n_real < pad_to and n_real >= pad_to - 2 * max(pad_multiple, 256):
        n_pad = pad_to - n_real
    elif pad_multiple and pad_multiple > 1 and n_real % pad_multiple:
        n_pad = pad_multiple - n_real % pad_multiple
    if n_pad:
        ids = torch.cat([ids, torch.zeros(n_pad, dtype=ids.dtype)])
        pos = torch.cat([pos, torch.arange(n_pad, dtype=torch.int32)])
        cu = torch.cat([cu, torch.tensor([n_real + n_pad], dtype=torch.int32)])
    from ..ops import _lib

    mv = lambda t: _lib.to_device(t, device)  # noqa: E731
    return PackedView(mv(ids), mv(pos), mv(cu), max(int(lens.max()) if B else 0, int(ids.numel()) - n_real), mv(pred_index), mv(targets.to(torch.int32)),
                      mv(grid_row), mv(grid_col), B, R, n_real)
