"""Pipeline parallelism: consecutive groups of decoder layers live on consecutive ranks; activations and their
gradients travel by point-to-point send/recv (NCCL on GPUs, gloo on CPU), as in the reference's Megatron backend
(``pipeline_model_parallel_size``, skyrl/backends/skyrl_train/workers/megatron/megatron_worker.py:469; schedules from
``get_forward_backward_func()``, megatron_model_wrapper.py:307,568; outputs collected from the last stage,
dispatch.py:35-42).  The schedule here is all-forward-then-all-backward over the micro-batches (GPipe): with the
packed, token-budgeted micro-batches this framework uses, the activation memory of the few in-flight micro-batches is
small next to 180 GB, and the bubble is (stages-1)/(micro-batches+stages-1) like 1F1B's.

Every pipeline rank sees the same packed micro-batches (token ids, positions, cu_seqlens), so tensor shapes are known
on both sides of every transfer and no shape handshake is needed.  Only the last stage evaluates the loss.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..models.decoder import CausalLM, ModelArgs, _EmbeddingFn
from ..ops import elementwise as ew


def stage_layer_range(num_layers: int, pp_size: int, pp_rank: int) -> Tuple[int, int]:
    """Contiguous layer range of a stage; earlier stages take the remainder layers."""
    base, rem = divmod(num_layers, pp_size)
    lo = pp_rank * base + min(pp_rank, rem)
    return lo, lo + base + (1 if pp_rank < rem else 0)


class PipelineStage(CausalLM):
    """The layers ``[lo, hi)`` of a model as their own ``CausalLM`` (own flat buffer, optimizer shard, checkpoints).
    Every stage keeps the embedding table slot of the layout (the first stage embeds, the last one uses it as a tied
    LM head); stages that need neither simply never touch it."""

    def __init__(self, full_args: ModelArgs, pp_rank: int, pp_size: int, group=None, device="cpu", dtype=torch.bfloat16,
                 seed: Optional[int] = 0):
        self.full_args, self.pp_rank, self.pp_size, self.group = full_args, pp_rank, pp_size, group
        self.lo, self.hi = stage_layer_range(full_args.num_layers, pp_size, pp_rank)
        super().__init__(dataclasses.replace(full_args, num_layers=self.hi - self.lo), device=device, dtype=dtype, seed=None)
        if seed is not None:
            self.load_from_full(CausalLM(full_args, device="cpu", dtype=torch.float32, seed=seed))

    @property
    def is_first(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    def _full_name(self, name: str) -> str:
        parts = name.split(".")
        if parts[0] == "layers":
            parts[1] = str(int(parts[1]) + self.lo)
        return ".".join(parts)

    @torch.no_grad()
    def load_from_full(self, full: CausalLM) -> None:
        for name, prm in self.named_flat_views():
            prm.copy_(full.p(self._full_name(name)).detach().to(prm.dtype))

    def stage_forward(self, input_ids, positions, cu_seqlens, max_seqlen: int, x_in: Optional[torch.Tensor]) -> torch.Tensor:
        """First stage: embeds ``input_ids``. Others: continue from ``x_in`` (the residual stream with every pending
        update already added).  Last stage returns final-normed hidden states, others the residual stream."""
        if self.is_first:
            x = _EmbeddingFn.apply(input_ids, self.p("embed"))
        else:
            x = x_in
        delta = None
        for i in range(self.args.num_layers):
            x, delta = self._layer(i, x, delta, positions, cu_seqlens, max_seqlen)
        if self.is_last:
            _, h = ew.add_rmsnorm(x, delta, self.p("final_norm"), self.args.rms_norm_eps)
            return h
        return x if delta is None else (x.float() + delta.float()).to(x.dtype)


def _peer(group, rank_in_group: int) -> int:
    return dist.get_global_rank(group, rank_in_group) if group is not None else rank_in_group


def pipeline_forward_backward(stage: PipelineStage, microbatches: Sequence[Dict[str, Any]],
                              loss_fn: Optional[Callable[[torch.Tensor, Dict[str, Any]], torch.Tensor]],
                              forward_only: bool = False) -> List[Optional[torch.Tensor]]:
    """Run all micro-batches through this rank's stage. ``microbatches[i]`` holds ``ids, pos, cu, max_seqlen`` (+ whatever
    ``loss_fn(hidden, mb)`` needs on the last stage).  Returns, on the last stage, the detached per-micro-batch loss
    values (or hidden states when ``forward_only`` and ``loss_fn`` is None); ``None`` entries elsewhere."""
    g = stage.group
    prev_r = _peer(g, stage.pp_rank - 1) if not stage.is_first else None
    next_r = _peer(g, stage.pp_rank + 1) if not stage.is_last else None
    H = stage.args.hidden_size
    dev, dt = stage.flat_params.device, stage.flat_params.dtype
    inputs: List[Optional[torch.Tensor]] = []
    outputs: List[torch.Tensor] = []
    results: List[Optional[torch.Tensor]] = []
    ctx = torch.no_grad() if forward_only else torch.enable_grad()
    with ctx:
        for mb in microbatches:
            x_in = None
            if prev_r is not None:
                x_in = torch.empty((mb["ids"].numel(), H), device=dev, dtype=dt)
                dist.recv(x_in, src=prev_r, group=g)
                if not forward_only:
                    x_in.requires_grad_()
            out = stage.stage_forward(mb["ids"], mb["pos"], mb["cu"], mb.get("max_seqlen", 0), x_in)
            if next_r is not None:
                dist.send(out.detach().contiguous(), dst=next_r, group=g)
                results.append(None)
            else:
                res = loss_fn(out, mb) if loss_fn is not None else out
                results.append(res.detach() if forward_only or loss_fn is None else res)
            inputs.append(x_in)
            outputs.append(out)
    if forward_only:
        return results
    # backward, last micro-batch first (frees its activations first)
    for i in reversed(range(len(microbatches))):
        if stage.is_last:
            results[i].backward()
            results[i] = results[i].detach()
        else:
            gout = torch.empty_like(outputs[i])
            dist.recv(gout, src=next_r, group=g)
            torch.autograd.backward(outputs[i], gout)
        if prev_r is not None:
            dist.send(inputs[i].grad.contiguous(), dst=prev_r, group=g)
        inputs[i], outputs[i] = None, None
    return results


def broadcast_from_last_stage(t: Optional[torch.Tensor], shape, dtype, stage: PipelineStage) -> torch.Tensor:
    """Make the last stage's result (log-probs, loss) available on every stage of the pipeline."""
    dev = stage.flat_params.device
    buf = t.contiguous() if stage.is_last else torch.empty(shape, device=dev, dtype=dtype)
    dist.broadcast(buf, src=_peer(stage.group, stage.pp_size - 1), group=stage.group)
    return buf
