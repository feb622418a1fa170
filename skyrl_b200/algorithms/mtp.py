"""Multi-token-prediction draft-head training: a decoupled soft cross-entropy that distils the trunk's next-next-token
distribution into a draft head on *detached* trunk features, with its own gradient clipping, so that speculative
decoding drafts stay on-policy without the draft loss touching the policy (reference: skyrl/backends/skyrl_train/mtp/
{soft_ce,hidden_capture,grad_clip}.py; config ``trainer.mtp``)."""

from __future__ import annotations

from typing import Iterable, Optional, Tuple

import torch


def soft_cross_entropy(student_logits: torch.Tensor, teacher_logits: torch.Tensor, mask: Optional[torch.Tensor] = None,
                       temperature: float = 1.0, chunk: int = 2048) -> torch.Tensor:
    """``-sum_v softmax(teacher)_v * log_softmax(student)_v`` averaged over unmasked rows; the teacher is detached.
    Rows are processed in chunks so that only ``chunk x V`` fp32 values are alive at a time."""
    T = student_logits.shape[0]
    total = student_logits.new_zeros((), dtype=torch.float32)
    denom = mask.float().sum().clamp_min(1.0) if mask is not None else torch.tensor(float(T), device=student_logits.device)
    for s in range(0, T, chunk):
        st = student_logits[s : s + chunk].float() / temperature
        te = teacher_logits[s : s + chunk].detach().float() / temperature
        row = -(torch.softmax(te, -1) * torch.log_softmax(st, -1)).sum(-1)
        if mask is not None:
            row = row * mask[s : s + chunk].float()
        total = total + row.sum()
    return total / denom


def mtp_draft_loss(draft_head, trunk_hidden: torch.Tensor, lm_head_weight: torch.Tensor, cu_seqlens: torch.Tensor,
                   loss_mask: Optional[torch.Tensor] = None, temperature: float = 1.0) -> torch.Tensor:
    """Draft head at position ``t`` sees the (detached) trunk state of ``t`` and predicts the trunk's distribution at
    ``t+1``.  Positions whose successor belongs to another packed sequence are masked out."""
    h = trunk_hidden.detach()
    T = h.shape[0]
    teacher = (h.float() @ lm_head_weight.detach().float().t())
    student = draft_head(h).float() @ lm_head_weight.detach().float().t()
    valid = torch.ones(T, dtype=torch.bool, device=h.device)
    valid[(cu_seqlens[1:] - 1).long()] = False  # last token of each sequence has no successor
    m = valid[:-1]
    if loss_mask is not None:
        m = m & loss_mask[1:].bool()
    return soft_cross_entropy(student[:-1], teacher[1:], m, temperature)


def clip_grad_norm_separately(params: Iterable[torch.nn.Parameter], max_norm: float) -> Tuple[float, float]:
    """Clip the draft head's gradients on their own norm (they must not share a budget with the policy's)."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return 0.0, 1.0
    norm = torch.sqrt(sum(g.float().pow(2).sum() for g in grads))
    coef = float(min(1.0, max_norm / (float(norm) + 1e-6)))
    if coef < 1.0:
        for g in grads:
            g.mul_(coef)
    return float(norm), coef


class DraftHead(torch.nn.Module):
    """Small residual MLP on the trunk state; its output goes through the (frozen, shared) LM head."""

    def __init__(self, hidden_size: int, expansion: int = 2, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.norm = torch.nn.LayerNorm(hidden_size, dtype=dtype, device=device)
        self.up = torch.nn.Linear(hidden_size, expansion * hidden_size, dtype=dtype, device=device)
        self.down = torch.nn.Linear(expansion * hidden_size, hidden_size, dtype=dtype, device=device)
        torch.nn.init.zeros_(self.down.weight)
        torch.nn.init.zeros_(self.down.bias)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        x = h.to(self.up.weight.dtype)
        return x + self.down(torch.nn.functional.silu(self.up(self.norm(x))))


def mtp_draft_backward(draft_head, trunk_hidden: torch.Tensor, lm_head_weight: torch.Tensor, cu_seqlens: torch.Tensor,
                       token_mask: Optional[torch.Tensor] = None, temperature: float = 1.0, scale: float = 1.0,
                       chunk: int = 1024) -> torch.Tensor:
    """Same loss as ``mtp_draft_loss`` (mean over the unmasked positions), evaluated and back-propagated in row chunks
    so that only ``chunk x V`` logits of the student and of the teacher exist at a time.  Gradients (times ``scale``)
    are accumulated into the draft head's parameters; returns the detached loss value.

    ``token_mask[t]`` (optional, ``[T]``): whether position ``t`` is a trained position; the pair (student at ``t``,
    teacher at ``t + 1``) counts when ``t + 1`` is trained and belongs to the same packed sequence."""
    h = trunk_hidden.detach()
    T = h.shape[0]
    W = lm_head_weight.detach().float()
    valid = torch.ones(T, dtype=torch.bool, device=h.device)
    valid[(cu_seqlens[1:] - 1).long()] = False
    m = valid[:-1]
    if token_mask is not None:
        m = m & token_mask[1:].bool()
    denom = m.float().sum().clamp_min(1.0)
    total = torch.zeros((), device=h.device, dtype=torch.float32)
    for s in range(0, T - 1, chunk):
        e = min(T - 1, s + chunk)
        mk = m[s:e]
        if not bool(mk.any()):
            continue
        with torch.no_grad():
            teacher = torch.softmax((h[s + 1 : e + 1].float() @ W.t()) / temperature, -1)
        student = torch.log_softmax((draft_head(h[s:e]).float() @ W.t()) / temperature, -1)
        part = (-(teacher * student).sum(-1) * mk.float()).sum() / denom
        (part * scale).backward()
        total = total + part.detach()
    return total
