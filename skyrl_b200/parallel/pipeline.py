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

    def replicated_ranges(self) -> List[Tuple[int, int]]:
        """Flat-buffer ranges whose gradient is identical on every stage after ``reduce_replicated_grads`` (the tied
        embedding table); they count once in the global gradient norm."""
        if not self.full_args.tie_word_embeddings:
            return []
        o, n = self.offsets["embed"]
        return [(o, o + n)]

    def reduce_replicated_grads(self) -> None:
        """Tied embeddings: the first stage's lookup gradient and the last stage's LM-head gradient are summed (the
        stages in between contribute zeros), so that every copy of the table takes the same update."""
        fg = getattr(self, "flat_main_grad", None)
        if self.pp_size == 1 or not self.full_args.tie_word_embeddings or fg is None:
            return
        o, n = self.offsets["embed"]
        dist.all_reduce(fg[o : o + n], group=self.group)

    def gather_full_state(self) -> Dict[str, torch.Tensor]:
        return PipelinedCausalLM(self).gather_full_state()

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


# ----------------------------------------------------------------------------- worker-facing wrapper
class _RelayFn(torch.autograd.Function):
    """Non-last stages: ship this stage's output to the next stage; in backward, receive its gradient from there.
    The value returned to the caller is a placeholder that carries the autograd edge (it has no numeric meaning)."""

    @staticmethod
    def forward(ctx, out, next_rank, group):
        ctx.next_rank, ctx.group, ctx.shape, ctx.dtype = next_rank, group, out.shape, out.dtype
        dist.send(out.detach().contiguous(), dst=next_rank, group=group)
        return out.new_zeros(())

    @staticmethod
    def backward(ctx, _g):
        gout = torch.empty(ctx.shape, dtype=ctx.dtype, device=_g.device)
        dist.recv(gout, src=ctx.next_rank, group=ctx.group)
        return gout, None, None


class PipelinedCausalLM:
    """What a worker needs from a pipeline-parallel policy: per-token log-probs of a packed batch on *every* rank of
    the pipeline group, with a backward pass that runs through all stages.

    Activations travel forward and gradients backward by send / recv; the last stage scores the tokens and broadcasts
    the log-probs, so the loss code runs identically on every stage.  On the last stage the log-probs are attached to
    the graph; on the others a zero-valued relay term carries the autograd edge, so that calling ``backward()`` on the
    (identical) loss of every rank drives the whole chain.  ``pred_logprobs`` moves one micro-batch through all stages;
    the worker's training and scoring loops use the ``_begin`` / ``_end`` halves to keep all stages busy."""

    def __init__(self, stage: PipelineStage):
        self.stage = stage

    def pred_logprobs(self, ids, pos, cu, max_seqlen, pred_index, targets, temp: float = 1.0, with_entropy: bool = False):
        return self.pred_logprobs_end(self.pred_logprobs_begin(ids, pos, cu, max_seqlen, pred_index, targets, temp,
                                                               with_entropy))

    def pred_logprobs_begin(self, ids, pos, cu, max_seqlen, pred_index, targets, temp: float = 1.0,
                            with_entropy: bool = False):
        """First half of ``pred_logprobs``: receive the previous stage's activations, run this stage, hand the result
        to the next stage (the last stage scores the tokens instead).  Nothing here waits for a later stage, so a
        caller that begins all its micro-batches before ending any keeps every stage busy: while stage ``s`` runs
        micro-batch ``k``, stage ``s - 1`` already runs ``k + 1`` (all-forward / all-backward schedule; the backward
        passes overlap the same way because each micro-batch's gradient hand-over is its own send / receive pair)."""
        st = self.stage
        g = st.group
        H = st.args.hidden_size
        dev, dt = st.flat_params.device, st.flat_params.dtype
        grad_on = torch.is_grad_enabled()
        x_in = None
        if not st.is_first:
            x_in = torch.empty((ids.numel(), H), device=dev, dtype=dt)
            dist.recv(x_in, src=_peer(g, st.pp_rank - 1), group=g)
            if grad_on:
                x_in.requires_grad_()
                prev = _peer(g, st.pp_rank - 1)
                x_in.register_hook(lambda gr: dist.send(gr.contiguous(), dst=prev, group=g))
        out = st.stage_forward(ids, pos, cu, max_seqlen, x_in)
        n = pred_index.numel()
        if st.is_last:
            lp, ent = st.token_logprobs(out[pred_index], targets, temp, with_entropy=with_entropy)
            return {"n": n, "lp": lp, "ent": ent}
        relay = _RelayFn.apply(out, _peer(g, st.pp_rank + 1), g) if grad_on else None
        if not grad_on:
            dist.send(out.detach().contiguous(), dst=_peer(g, st.pp_rank + 1), group=g)
        return {"n": n, "relay": relay}

    def pred_logprobs_end(self, h):
        """Second half: the last stage's log-probs (and entropies) reach every stage of the pipeline."""
        st = self.stage
        g = st.group
        dev = st.flat_params.device
        n = h["n"]
        last = _peer(g, st.pp_size - 1)
        if st.is_last:
            lp, ent = h["lp"], h["ent"]
            # row 0: log-probs, row 1: entropies; the extra column says whether entropies were computed at all
            pack = torch.zeros((2, n + 1), device=dev, dtype=torch.float32)
            pack[0, :n] = lp.detach().float()
            if ent is not None:
                pack[1, :n] = ent.detach().float()
                pack[1, n] = 1.0
            dist.broadcast(pack, src=last, group=g)
            return lp, ent
        pack = torch.empty((2, n + 1), device=dev, dtype=torch.float32)
        dist.broadcast(pack, src=last, group=g)
        lp = pack[0, :n]
        ent = pack[1, :n] if bool(pack[1, n] > 0) else None
        if h.get("relay") is not None:
            lp = lp + h["relay"]  # numerically a no-op; gives this rank's loss a path into its stage
        return lp, ent

    @torch.no_grad()
    def gather_full_state(self) -> Dict[str, torch.Tensor]:
        """Every stage's parameters on every rank, keyed by the unsharded model's names."""
        st = self.stage
        out: Dict[str, torch.Tensor] = {}
        for r in range(st.pp_size):
            names = [None]
            if r == st.pp_rank:
                names = [[(st._full_name(n), tuple(p.shape)) for n, p in st.named_flat_views()]]
            dist.broadcast_object_list(names, src=_peer(st.group, r), group=st.group)
            own = dict(st.named_flat_views()) if r == st.pp_rank else {}
            lo, _ = stage_layer_range(st.full_args.num_layers, st.pp_size, r)
            for full_name, shape in names[0]:
                if r == st.pp_rank:
                    parts = full_name.split(".")
                    local = full_name if parts[0] != "layers" else ".".join(["layers", str(int(parts[1]) - lo)] + parts[2:])
                    t = own[local].detach().contiguous()
                else:
                    t = torch.empty(shape, device=st.flat_params.device, dtype=st.flat_params.dtype)
                dist.broadcast(t, src=_peer(st.group, r), group=st.group)
                is_layer = full_name.startswith("layers.")
                first_owner = full_name == "embed" and r == 0
                last_owner = full_name in ("final_norm", "lm_head") and r == st.pp_size - 1
                if is_layer or first_owner or last_owner:
                    out[full_name] = t
        return out
