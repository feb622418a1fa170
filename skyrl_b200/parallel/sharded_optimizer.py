"""ZeRO-style sharded AdamW over the model's flat parameter / gradient buffers.

Every rank computes with the full bf16 parameter buffer (the models targeted here fit one B200 many
times over) while the fp32 master weights and both Adam moments are sharded 1/world per rank.  One
optimizer step is

    reduce-scatter(grad)  ->  global-norm clip  ->  AdamW on the owned shard  ->  all-gather(bf16 params)

which is exactly the traffic FSDP2 generates for the reference
(skyrl/backends/skyrl_train/distributed/fsdp_strategy.py:152-186, fsdp_utils.py:209-251), but it is
issued once per step on one flat range instead of per layer.  Two transports implement it:

* ``peer``  - the fused kernels of ``csrc/comm.cu``: each rank pulls its gradient range from every
  peer's buffer over NVLink, reduces in registers, applies AdamW and stores the new bf16
  parameters straight into every peer's parameter buffer (which is also what the colocated
  generation engines read, so the same stores are the trainer->rollout weight sync);
* ``nccl``  - ``reduce_scatter_tensor`` / ``all_gather_into_tensor``: the measured baseline and the
  CPU (gloo) path.

The step skips the update when the gradient norm is not finite, like the reference.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import optim as optim_ops


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class ShardedAdamW:
    def __init__(self, flat_params: torch.Tensor, flat_grads: torch.Tensor, lr: float = 1e-6, betas=(0.9, 0.999),
                 eps: float = 1e-8, weight_decay: float = 0.01, max_grad_norm: float = 1.0,
                 group: Optional[dist.ProcessGroup] = None, transport: str = "auto", peer_ctx=None,
                 numel: Optional[int] = None, params_symm=None, grads_symm=None, norm_group=None,
                 dup_ranges=None, count_dups: bool = True, replica_group: Optional[dist.ProcessGroup] = None):
        """``norm_group`` / ``dup_ranges`` / ``count_dups`` serve tensor parallelism: the gradient norm is also summed
        over ``norm_group`` (the TP group), and the flat-buffer ranges listed in ``dup_ranges`` (parameters replicated
        across that group) enter the norm on one rank only (``count_dups``).

        ``replica_group`` enables hybrid sharding (the reference's HSDP mesh ``ddp x fsdp``, fsdp_utils.py:254-261):
        optimizer state is sharded over ``group`` only, and ranks that hold the same shard in different groups sum
        their reduced gradients over ``replica_group`` before the (identical) update."""
        self.group = group
        self.replica_group = replica_group
        self.norm_group, self.dup_ranges, self.count_dups = norm_group, list(dup_ranges or []), count_dups
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.params = flat_params
        self.grads = flat_grads
        self.numel = numel if numel is not None else flat_params.numel()
        assert flat_params.numel() == flat_grads.numel()
        assert flat_params.numel() % (self.world * 8) == 0, "flat buffers must be padded to a multiple of 8 * world"
        self.shard = flat_params.numel() // self.world
        self.lo = self.rank * self.shard
        dev = flat_params.device
        self.master = flat_params[self.lo : self.lo + self.shard].float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.lr, self.betas, self.eps, self.weight_decay = lr, tuple(betas), eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self._sq = torch.zeros(1, device=dev, dtype=torch.float32)
        self._coef = torch.ones(1, device=dev, dtype=torch.float32)
        self._skip = torch.zeros(1, device=dev, dtype=torch.int32)
        self._norm = torch.zeros(1, device=dev, dtype=torch.float32)
        self._grad_shard = torch.zeros(self.shard, device=dev, dtype=torch.float32) if self.world > 1 else None
        self.params_symm, self.grads_symm = params_symm, grads_symm
        if transport == "auto":
            transport = "peer" if (peer_ctx is not None and self.world > 1 and params_symm is not None
                                   and grads_symm is not None) else "nccl"
        self.transport = transport
        self.peer_ctx = peer_ctx
        self.last_grad_norm: Optional[torch.Tensor] = None
        self._buckets_done: list = []
        self._side = torch.cuda.Stream(device=dev) if (transport == "peer" and dev.type == "cuda") else None

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> torch.Tensor:
        """Apply one update; returns the (pre-clip) global gradient norm as a device scalar."""
        self.step_count += 1
        b1, b2 = self.betas
        if self.world > 1 and self.transport == "peer":
            # peer-memory path: loads from every peer's gradient buffer, AdamW, stores into every peer's parameters
            ctx = self.peer_ctx
            if self._buckets_done:
                # part of the reduce-scatter already ran behind the backward pass (``reduce_bucket``): wait for it, then
                # reduce what is left (the embedding range and anything whose hook did not fire)
                torch.cuda.current_stream().wait_stream(self._side)
                done = sorted(self._buckets_done)
                rest, cur = [], 0
                for (a, b) in done:
                    if a > cur:
                        rest.append((cur, a))
                    cur = max(cur, b)
                if cur < self.params.numel():
                    rest.append((cur, self.params.numel()))
                ctx.finish_reduce(self.grads_symm, self._grad_shard, self.lo, self.shard, rest, first=False)
                self._buckets_done = []
            else:
                ctx.reduce_scatter_and_norm(self.grads_symm, self._grad_shard, self.lo, self.shard)
            norm, skipped = ctx.adamw_and_push(self.master, self.exp_avg, self.exp_avg_sq, self._grad_shard,
                                               self.params_symm, self.lo, self.shard, self.lr, b1, b2, self.eps,
                                               self.weight_decay, self.step_count, self.max_grad_norm, grad_scale)
            self.last_grad_norm = norm.clone()
            return self.last_grad_norm
        if self.world == 1:
            g = self.grads
        else:
            dist.reduce_scatter_tensor(self._grad_shard, self.grads, op=dist.ReduceOp.SUM, group=self.group)
            g = self._grad_shard
        if self.replica_group is not None and dist.get_world_size(self.replica_group) > 1:
            if g is self.grads:
                g = self.grads  # one-rank shard group: the whole gradient is "the shard"
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.replica_group)
        self._sq.zero_()
        optim_ops.sqnorm_accum(g, self._sq)
        if self.dup_ranges and not self.count_dups:
            dup = torch.zeros_like(self._sq)
            for r_lo, r_hi in self.dup_ranges:  # intersect with this rank's optimizer shard
                s0, s1 = max(r_lo, self.lo) - self.lo, min(r_hi, self.lo + self.shard) - self.lo
                if s1 > s0:
                    s4 = (s0 + 3) // 4 * 4  # the norm kernel reads 16-byte vectors
                    if s4 > s0:
                        dup += g[s0 : min(s4, s1)].float().pow(2).sum()
                    if s1 > s4:
                        optim_ops.sqnorm_accum(g[s4:s1], dup)
            self._sq -= dup
        if self.world > 1:
            dist.all_reduce(self._sq, op=dist.ReduceOp.SUM, group=self.group)
        if self.norm_group is not None and dist.get_world_size(self.norm_group) > 1:
            dist.all_reduce(self._sq, op=dist.ReduceOp.SUM, group=self.norm_group)
        optim_ops.clip_coef(self._sq, self.max_grad_norm, grad_scale, self._coef, self._skip, self._norm)
        shard_params = self.params[self.lo : self.lo + self.shard]
        optim_ops.adamw_flat(self.master, self.exp_avg, self.exp_avg_sq, g, shard_params, self.lr, b1, b2, self.eps,
                             self.weight_decay, self.step_count, self._coef, self._skip)
        if self.world > 1:
            dist.all_gather_into_tensor(self.params, shard_params.clone(), group=self.group)
        self.last_grad_norm = self._norm.clone()
        return self.last_grad_norm

    # ------------------------------------------------------------------ reduce-scatter behind the backward pass
    @property
    def can_overlap_reduce(self) -> bool:
        return self.world > 1 and self.transport == "peer" and self._side is not None

    def reduce_bucket(self, lo: int, hi: int) -> None:
        """Gradients of flat range ``[lo, hi)`` are final on this rank (called from a backward hook during the last
        micro-batch before ``step``): reduce this rank's part of the range on a side stream while the backward pass of
        the earlier layers keeps running.  Every rank must call this for the same ranges in the same order."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        with torch.cuda.stream(self._side):
            self._side.wait_event(ev)
            self.peer_ctx.reduce_scatter_bucket(self.grads_symm, self._grad_shard, self.lo, self.shard, lo, hi,
                                                first=not self._buckets_done)
        self._buckets_done.append((lo, hi))

    def zero_grad(self) -> None:
        self.grads.zero_()

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        return {"master": self.master, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "step": self.step_count,
                "lr": self.lr, "world_size": self.world, "rank": self.rank, "shard": self.shard}

    def load_state_dict(self, sd: dict) -> None:
        if sd["world_size"] != self.world or sd["shard"] != self.shard:
            raise ValueError(f"optimizer shard saved for world size {sd['world_size']} cannot be loaded into world size "
                             f"{self.world}")
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.step_count = int(sd["step"])
        self.lr = float(sd.get("lr", self.lr))

    def offload(self) -> None:
        """Move optimizer state to pinned host memory (colocation: frees HBM while the engine runs)."""
        for name in ("master", "exp_avg", "exp_avg_sq"):
            t = getattr(self, name)
            if t.is_cuda:
                host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                host.copy_(t, non_blocking=True)
                setattr(self, name, host)
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def backload(self) -> None:
        dev = self.params.device
        for name in ("master", "exp_avg", "exp_avg_sq"):
            t = getattr(self, name)
            if t.device != dev:
                setattr(self, name, t.to(dev, non_blocking=True))

    def resync_master_from_params(self) -> None:
        """After loading bf16 weights directly into the parameter buffer."""
        self.master.copy_(self.params[self.lo : self.lo + self.shard].float())


def get_scheduler(name: str, optimizer: ShardedAdamW, num_warmup_steps: int = 0, num_training_steps: Optional[int] = None,
                  base_lr: Optional[float] = None):
    """LR schedules by HF name: constant, constant_with_warmup, linear, cosine."""
    base = base_lr if base_lr is not None else optimizer.lr

    def factor(step: int) -> float:
        warm = min(1.0, (step + 1) / num_warmup_steps) if num_warmup_steps > 0 else 1.0
        if name in ("constant", "constant_with_warmup"):
            return warm if name == "constant_with_warmup" else 1.0
        total = max(1, (num_training_steps or 1) - num_warmup_steps)
        prog = min(1.0, max(0.0, (step - num_warmup_steps) / total))
        if step < num_warmup_steps:
            return warm
        if name == "linear":
            return 1.0 - prog
        if name == "cosine":
            return 0.5 * (1.0 + math.cos(math.pi * prog))
        raise ValueError(f"unknown scheduler '{name}'")

    class _Sched:
        def __init__(self):
            self.last_step = 0
            optimizer.set_lr(base * factor(0))

        def step(self):
            self.last_step += 1
            optimizer.set_lr(base * factor(self.last_step))

        def state_dict(self):
            return {"last_step": self.last_step}

        def load_state_dict(self, sd):
            self.last_step = sd["last_step"]
            optimizer.set_lr(base * factor(self.last_step))

        def get_last_lr(self):
            return [optimizer.lr]

    return _Sched()
