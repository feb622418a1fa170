"""Training workers: policy, critic and reference model replicas running SPMD, one process per GPU.

The verbs are the reference's (skyrl/backends/skyrl_train/workers/worker.py:831-1639):
``forward`` (log-probs or values, no grad), ``forward_backward`` (micro-batch loop with gradient
accumulation), ``optim_step``, ``set_lr``, checkpoint verbs, offload/backload.  What differs is
where the work happens: a worker receives *its own shard* of the batch (built on the same rank by
the controller), packs it to tokens, runs the packed model, and reads log-probabilities from the
fused LM-head kernel only at the positions that predict response tokens.  Gradients accumulate into
one flat fp32 buffer that the sharded optimizer reduces across ranks once per step, so there is no
per-layer collective and no ``dp_size`` loss-scaling trick: ranks *sum* their pre-scaled losses.
"""

from __future__ import annotations

import ctypes
import math
import os
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..algorithms import rl
from ..models.decoder import CausalLM, build_model
from ..ops import _lib
from ..parallel.dist import DistEnv, get_env
from ..parallel.sharded_optimizer import ShardedAdamW, get_scheduler
from ..train.batch import TrainingInputBatch, TrainingOutputBatch
from ..train.preprocess import PackedView, pack_batch
from ..utils.torch_utils import masked_mean


# ----------------------------------------------------------------------------- micro-batching
def microbatch_indices(seq_lens: Sequence[int], micro_batch_size: int, max_tokens: int, packing: str = "balanced") -> List[List[int]]:
    """Row-index groups: by token budget (C++ runtime) when ``max_tokens > 0``, else by count.  ``packing``:
    ``balanced`` = equal-load bins; ``full`` = first-fit-decreasing, i.e. every bin but the last is filled to the
    budget, which makes the packed length -- and with it every activation size -- the same from micro-batch to
    micro-batch and from step to step.

    Reference: ``max_tokens_per_microbatch`` / ``micro_*_batch_size_per_gpu`` handling in
    skyrl/backends/skyrl_train/workers/worker_utils.py:248-444.
    """
    n = len(seq_lens)
    if n == 0:
        return []
    if max_tokens is not None and max_tokens > 0:
        lens = np.asarray(seq_lens, dtype=np.int32)
        budget = max(int(max_tokens), int(lens.max()))
        out = np.zeros(n, dtype=np.int32)
        rt = _lib.runtime()
        fn = rt.sbrt_ffd_pack if packing == "full" else rt.sbrt_balanced_bins
        fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        bins = fn(lens.ctypes.data, n, budget, out.ctypes.data)
        groups: List[List[int]] = [[] for _ in range(bins)]
        for i, b in enumerate(out.tolist()):
            groups[b].append(i)
        return [g for g in groups if g]
    mbs = max(1, micro_batch_size)
    return [list(range(s, min(n, s + mbs))) for s in range(0, n, mbs)]


def sync_num_microbatches(n_local: int, env: DistEnv, group=None) -> int:
    """Ranks whose model forward contains collectives (one tensor / sequence / expert / pipeline group) must run the
    same number of micro-batches: take the MAX over ``group``.  Reference: worker_utils.py:343-357, which pads over
    the whole world because FSDP2 gathers parameters in every forward; here plain data-parallel ranks share nothing
    until the optimizer step, so they are never padded (``group=None`` with no model-parallel mesh)."""
    if not dist.is_initialized() or env.world_size == 1:
        return n_local
    t = torch.tensor([n_local], device=env.device, dtype=torch.int64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t.item())


def materialize_metrics(metrics_list: List[Dict[str, Any]]) -> List[Dict[str, float]]:
    """Per-micro-batch metric dicts may hold 0-dim device tensors; bring all of them to the host with ONE copy (one
    device synchronisation per mini-batch instead of several per micro-batch)."""
    slots = [(i, k) for i, m in enumerate(metrics_list) for k, v in m.items() if isinstance(v, torch.Tensor)]
    if not slots:
        return metrics_list
    vals = _lib.to_host(torch.stack([metrics_list[i][k].detach().float().reshape(()) for i, k in slots])).tolist()
    out = [dict(m) for m in metrics_list]
    for (i, k), v in zip(slots, vals):
        out[i][k] = float(v)
    return out


def reduce_metrics(metrics_list: List[Dict[str, float]]) -> Dict[str, float]:
    """Combine per-micro-batch metrics: ``*_loss`` / ``loss`` summed, ``*_min`` / ``*_max`` min/max, others averaged."""
    if not metrics_list:
        return {}
    keys = set().union(*[m.keys() for m in metrics_list])
    out = {}
    for k in keys:
        vals = [m[k] for m in metrics_list if k in m and isinstance(m[k], (int, float))]
        if not vals:
            continue
        if k.endswith("_min"):
            out[k] = min(vals)
        elif k.endswith("_max"):
            out[k] = max(vals)
        elif k.endswith("loss") or k.endswith("_loss_sum"):
            out[k] = float(sum(vals))
        else:
            out[k] = float(sum(vals) / len(vals))
    return out


def all_reduce_metrics(metrics: Dict[str, float], env: DistEnv) -> Dict[str, float]:
    if not dist.is_initialized() or env.world_size == 1 or not metrics:
        return metrics
    keys = sorted(metrics)
    sums = torch.tensor([metrics[k] for k in keys], device=env.device, dtype=torch.float64)
    mins, maxs = sums.clone(), sums.clone()
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    dist.all_reduce(mins, op=dist.ReduceOp.MIN)
    dist.all_reduce(maxs, op=dist.ReduceOp.MAX)
    out = {}
    for i, k in enumerate(keys):
        if k.endswith("_min"):
            out[k] = float(mins[i])
        elif k.endswith("_max"):
            out[k] = float(maxs[i])
        elif k.endswith("loss") or k.endswith("_loss_sum"):
            out[k] = float(sums[i])
        else:
            out[k] = float(sums[i]) / env.world_size
    return out


class DeviceWaitError(RuntimeError):
    """A kernel's bounded wait (mbarrier, peer flag, barrier epoch) ran out; see ``csrc/ptx.cuh`` for the codes."""


# ----------------------------------------------------------------------------- worker
class ModelWorker:
    role = "model"

    def __init__(self, cfg, model: Optional[CausalLM] = None, model_path: Optional[str] = None, env: Optional[DistEnv] = None,
                 trainable: bool = True, value_head: bool = False, optimizer_cfg=None, peer_ctx=None,
                 flat_buffer: Optional[torch.Tensor] = None, flat_grad: Optional[torch.Tensor] = None, seed: int = 0):
        self.cfg = cfg  # TrainerConfig
        self.env = env or get_env()
        dev = self.env.device
        dtype = torch.bfloat16 if (cfg.bf16 and dev.type == "cuda") else torch.float32
        self.params_symm = self.grads_symm = None
        self._replay_on = False
        self.mesh = None
        self.expert_parallel = self.sequence_parallel = False
        tp_size = self._tp_size_from_cfg(cfg)
        if tp_size > 1 and model is None:
            # Megatron-style strategy: tensor-parallel shards inside groups of consecutive ranks, data parallel across
            from ..models.decoder import resolve_model_args
            from ..models.tp_decoder import TPCausalLM
            from ..parallel.dist import build_mesh
            from ..parallel.peer import PeerContext
            from ..parallel.tensor_parallel import TPGroup

            self.mesh = build_mesh(tp_size, self.env)
            tp_peer = PeerContext(dev, group=self.mesh.tp_group) if dev.type == "cuda" else None
            self.tp = TPGroup(tp_peer, self.mesh.tp_group)
            margs = resolve_model_args(model_path)
            model = TPCausalLM(margs, self.tp, device=dev, dtype=dtype, seed=None, value_head=value_head,
                               vocab_parallel_head=bool(getattr(cfg.b200, "vocab_parallel_lm_head", False)))
            from ..models.decoder import PRESETS

            if model_path in PRESETS and dev.type == "cuda" and model.num_parameters() * tp_size > 2_000_000_000:
                model.init_random_on_device(seed)  # multi-billion-parameter presets: no fp32 host copy per rank
            else:
                full = build_model(model_path, device="cpu", dtype=torch.float32, seed=seed, value_head=value_head)
                model.load_from_full(full)
                del full
            peer_ctx = None  # the flat-buffer peer optimizer spans the whole world; TP uses the DP group over NCCL
        pp_size = self._pp_size_from_cfg(cfg) if (model is None and tp_size == 1) else 1
        self.pipe = None
        if pp_size > 1:
            # consecutive ranks hold consecutive layer ranges; one data shard per pipeline group
            from ..models.decoder import resolve_model_args
            from ..parallel.dist import build_mesh
            from ..parallel.pipeline import PipelinedCausalLM, PipelineStage

            if value_head:
                raise NotImplementedError("the critic runs without pipeline parallelism")
            self.mesh = build_mesh(pp_size, self.env)
            model = PipelineStage(resolve_model_args(model_path), self.mesh.tp_rank, pp_size, group=self.mesh.tp_group,
                                  device=dev, dtype=dtype, seed=None)
            full = build_model(model_path, device="cpu", dtype=torch.float32, seed=seed)
            model.load_from_full(full)
            del full
            self.pipe = PipelinedCausalLM(model)
            peer_ctx = None
        ep_size = self._ep_size_from_cfg(cfg) if (model is None and tp_size == 1) else 1
        self.expert_parallel = ep_size > 1
        if self.expert_parallel:
            # experts sharded over groups of consecutive ranks; tokens stay data parallel on every rank
            from ..models.decoder import resolve_model_args
            from ..models.tp_decoder import EPCausalLM
            from ..parallel.dist import build_mesh
            from ..parallel.peer import PeerContext
            from ..parallel.tensor_parallel import TPGroup

            if value_head:
                raise NotImplementedError("the critic runs without expert parallelism")
            self.mesh = build_mesh(ep_size, self.env)
            ep_peer = PeerContext(dev, group=self.mesh.tp_group) if dev.type == "cuda" else None
            self.tp = TPGroup(ep_peer, self.mesh.tp_group)
            model = EPCausalLM(resolve_model_args(model_path), self.tp, device=dev, dtype=dtype, seed=None)
            from ..models.decoder import PRESETS

            if model_path in PRESETS and dev.type == "cuda" and model.num_parameters() > 2_000_000_000:
                model.init_random_on_device(seed)
            else:
                full = build_model(model_path, device="cpu", dtype=torch.float32, seed=seed)
                model.load_from_full(full)
                del full
            peer_ctx = None
        use_peer = peer_ctx is not None and trainable and self.env.world_size > 1 and dev.type == "cuda"
        sp_size = self._sp_size_from_cfg(cfg) if model is None and tp_size == 1 else 1
        self.sequence_parallel = sp_size > 1
        if model is None:
            if use_peer:
                from ..models.decoder import flat_numel_for, resolve_model_args

                n = flat_numel_for(resolve_model_args(model_path), value_head)
                self.params_symm = peer_ctx.alloc(n, dtype)
                self.grads_symm = peer_ctx.alloc(n, torch.float32)
                flat_buffer, flat_grad = self.params_symm.local, self.grads_symm.local
            lora_cfg = getattr(getattr(cfg, self.role, cfg.policy).model, "lora", None) if self.role in ("policy", "critic") else None
            use_lora = trainable and not value_head and lora_cfg is not None and lora_cfg.rank > 0
            if use_lora and use_peer:
                use_peer, flat_buffer, flat_grad = False, None, None  # adapter buffers are small: plain NCCL reduction
                self.params_symm = self.grads_symm = None
                peer_ctx = None
            model = build_model(model_path, device=dev, dtype=dtype, value_head=value_head, seed=seed,
                                flat_buffer=flat_buffer)
            if use_lora:
                from ..models.lora import LoRACausalLM

                if sp_size > 1:
                    raise NotImplementedError("LoRA together with sequence parallelism is not supported")
                model = LoRACausalLM(model.args, rank=lora_cfg.rank, alpha=lora_cfg.alpha, dropout=lora_cfg.dropout,
                                     target_modules=lora_cfg.target_modules, exclude_modules=lora_cfg.exclude_modules,
                                     init_method=lora_cfg.init_method, device=dev, dtype=dtype,
                                     flat_buffer=model.flat_params, seed=None, lora_seed=seed + 1)
            if self.sequence_parallel:
                # Ulysses: same (replicated) parameters, sequence-sharded forward; groups of consecutive ranks
                from ..models.tp_decoder import UlyssesCausalLM
                from ..parallel.dist import build_mesh
                from ..parallel.peer import PeerContext
                from ..parallel.tensor_parallel import TPGroup

                self.mesh = build_mesh(sp_size, self.env)
                sp_peer = PeerContext(dev, group=self.mesh.tp_group) if dev.type == "cuda" else None
                self.tp = TPGroup(sp_peer, self.mesh.tp_group)
                self._plain_model = model
                cls = UlyssesCausalLM
                if self._sp_backend(cfg) == "context":
                    from ..models.tp_decoder import ContextParallelCausalLM as cls  # noqa: N813
                model = cls(model.args, self.tp, device=dev, dtype=dtype, flat_buffer=model.flat_params, seed=None,
                            value_head=value_head)
        self.model = model
        qcfg = getattr(cfg.policy.model, "fake_int4_qat", None)
        if trainable and qcfg is not None and qcfg.enabled:
            self.model.fake_int4_qat = qcfg  # MoE expert weights are fake-quantised in the training forward
        self.model.gradient_checkpointing = bool(cfg.gradient_checkpointing) and trainable
        self.trainable = trainable
        self.optimizer: Optional[ShardedAdamW] = None
        self.scheduler = None
        self._on_device = True
        self._offloaded: Dict[str, torch.Tensor] = {}
        self.num_microbatches_accumulated = 0
        if trainable:
            ocfg = optimizer_cfg
            if flat_grad is None:
                flat_grad = torch.zeros(model.flat_params.numel(), device=dev, dtype=torch.float32)
            model.attach_main_grad(flat_grad)
            self.flat_grad = flat_grad
            extra = {}
            # sequence parallelism replicates every parameter and each rank of the group back-propagates only its
            # token shard, so the gradient is complete only after a sum over *all* ranks: the optimizer then spans the
            # world exactly as in plain data parallelism (fused peer transport included)
            if self.mesh is not None and not self.sequence_parallel:
                from ..models.tp_decoder import REPLICATED_LEAVES

                if self.expert_parallel or self.pipe is not None:
                    dups = model.replicated_ranges()
                else:
                    rep = getattr(model, "replicated_leaves", REPLICATED_LEAVES)
                    dups = [(o, o + n) for name, (o, n) in model.offsets.items() if name.split(".")[-1] in rep]
                extra = dict(group=self.mesh.dp_group, transport="nccl", norm_group=self.mesh.tp_group, dup_ranges=dups,
                             count_dups=self.mesh.tp_rank == 0)
            node = {"policy": cfg.policy, "critic": cfg.critic}.get(self.role, cfg.policy)
            fsdp_size = int(getattr(getattr(node, "fsdp_config", None), "fsdp_size", -1) or -1)
            if self.mesh is None and 0 < fsdp_size < self.env.world_size and dist.is_initialized():
                # hybrid sharding: optimizer state sharded inside groups of fsdp_size ranks, replicated across them
                from ..parallel.dist import build_hsdp_groups

                shard_g, replica_g = build_hsdp_groups(fsdp_size, self.env)
                extra = dict(group=shard_g, replica_group=replica_g, transport="nccl")
                peer_ctx = None
            self.optimizer = ShardedAdamW(model.flat_params, flat_grad, lr=ocfg.lr, betas=tuple(ocfg.adam_betas),
                                          weight_decay=ocfg.weight_decay, max_grad_norm=ocfg.max_grad_norm,
                                          peer_ctx=peer_ctx, params_symm=self.params_symm, grads_symm=self.grads_symm,
                                          **extra)
            self.scheduler = get_scheduler(ocfg.scheduler, self.optimizer, ocfg.num_warmup_steps, base_lr=ocfg.lr)

    # ------------------------------------------------------------------ helpers
    def _max_tokens(self) -> int:
        return int(self.cfg.max_tokens_per_microbatch or -1)

    def _num_microbatches(self, n_local: int) -> int:
        """Micro-batches this rank runs: its own count in plain data parallelism; the maximum over the model-parallel
        group otherwise (its members hold the same batch, but expert-parallel members hold different ones)."""
        if self.mesh is None:
            return n_local
        return sync_num_microbatches(n_local, self.env, group=self.mesh.tp_group)

    def check_device_status(self, where: str) -> None:
        """Raise when a bounded device-side wait gave up since the last check (a peer that never reached a barrier, a
        copy that never landed).  Synchronises the device, so it is called where the host reads results anyway."""
        if self.env.device.type != "cuda":
            return
        code = _lib.status_read_clear()
        if code != 0:
            raise DeviceWaitError(f"{self.role} worker, rank {self.env.rank}: a device-side wait timed out during {where} "
                                  f"(status 0x{code:x}); the step's results are incomplete and nothing was published")

    def _seq_lens(self, batch: TrainingInputBatch) -> List[int]:
        return batch["attention_mask"].sum(1).tolist()

    def _pack(self, batch: TrainingInputBatch, rows: List[int]) -> PackedView:
        idx = torch.tensor(rows, dtype=torch.long)
        b2 = self.cfg.b200
        pv = pack_batch(batch["sequences"][idx], batch["attention_mask"][idx], batch["response_mask"][idx],
                        self.env.device, pad_multiple=int(getattr(b2, "pack_pad_multiple", 0) or 0),
                        pad_to=self._max_tokens() if getattr(b2, "microbatch_packing", "balanced") == "full" else 0)
        routes = batch.get("rollout_expert_indices")
        if routes is not None and self._replays_routing():
            # rollout-time expert choices of the packed tokens; the dummy tail that pads the pack keeps its own routing
            att = batch["attention_mask"][idx].cpu().bool()
            packed = routes[idx][att]
            tail = int(pv.ids.numel()) - packed.shape[0]
            if tail:
                packed = torch.cat([packed, packed.new_full((tail, *packed.shape[1:]), -1)], 0)
            pv.routing = _lib.to_device(packed, self.env.device)
        return pv

    def _replays_routing(self) -> bool:
        """Router replay (reference: utils/replay_utils.py, ``megatron_config.moe_enable_routing_replay``): the policy
        and the reference model run their mixture-of-experts layers through the experts the rollout engine chose."""
        if self.role not in ("policy", "ref") or not self.model.args.num_experts or getattr(self, "pipe", None) is not None:
            return False
        node = self.cfg.policy if self.role == "policy" else self.cfg.ref
        return bool(getattr(getattr(node, "megatron_config", None), "moe_enable_routing_replay", False))

    def _rows_to_device(self, t: Optional[torch.Tensor], rows: List[int]) -> Optional[torch.Tensor]:
        if t is None:
            return None
        return _lib.to_device(t[torch.tensor(rows, dtype=torch.long)], self.env.device)

    def _hidden(self, pv: PackedView) -> torch.Tensor:
        if pv.routing is not None or self._replay_on:
            # stays set through the backward pass (checkpointed layers route again when they are recomputed); the next
            # micro-batch replaces it and the end of the pass clears it
            from ..models import router_replay

            router_replay.set_replay(pv.routing)
            self._replay_on = pv.routing is not None
        return self.model(pv.ids, pv.positions, pv.cu_seqlens, pv.max_seqlen)

    def _end_replay(self) -> None:
        if self._replay_on:
            from ..models import router_replay

            router_replay.set_replay(None)
            self._replay_on = False

    # ------------------------------------------------------------------ profiling verbs (reference: worker.py:361-457)
    def start_profile(self) -> None:
        from ..utils.profiler import Profiler

        node = {"policy": self.cfg.policy, "critic": self.cfg.critic, "ref": self.cfg.ref}.get(self.role, self.cfg.policy)
        pcfg = getattr(node, "torch_profiler_config", None)
        if pcfg is None or not pcfg.enable:
            self._profiler = None
            return
        self._profiler = Profiler(pcfg, self.env.rank)
        self._profiler.start()

    def profile_step(self) -> None:
        p = getattr(self, "_profiler", None)
        if p is not None:
            p.step()

    def stop_profile(self) -> Optional[str]:
        p = getattr(self, "_profiler", None)
        if p is None:
            return None
        p.stop()
        return p.kernel_summary()

    def record_memory_history(self, enabled: bool = True) -> None:
        if torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=100000 if enabled else None)

    def dump_memory_snapshot(self, out_dir: str, tag: str = "") -> Optional[str]:
        """Pickled allocator snapshot of this rank (viewable with pytorch.org/memory_viz)."""
        if not torch.cuda.is_available():
            return None
        os.makedirs(out_dir, exist_ok=True)
        path = os.path.join(out_dir, f"memory_{self.role}_rank{self.env.rank}{('_' + tag) if tag else ''}.pickle")
        torch.cuda.memory._dump_snapshot(path)
        return path

    def _sp_size_from_cfg(self, cfg) -> int:
        node = {"policy": cfg.policy, "ref": cfg.ref, "critic": cfg.critic}.get(self.role, cfg.policy)
        if getattr(cfg, "strategy", "fsdp") == "megatron":
            # Megatron naming: context parallelism shards the sequence (tensor / expert / pipeline sizes are handled
            # by their own branches before this one is reached)
            mc = getattr(node, "megatron_config", None)
            return int(getattr(mc, "context_parallel_size", 1) or 1)
        return int(getattr(node, "sequence_parallel_size", 1) or 1)

    @staticmethod
    def _sp_backend(cfg) -> str:
        """``ulysses`` (heads exchanged by all-to-all; degree divides the key/value heads) or ``context`` (keys and
        values all-gathered; any degree)."""
        if getattr(cfg, "strategy", "fsdp") == "megatron":
            return "context"
        b = str(getattr(cfg, "sequence_parallel_backend", "ulysses") or "ulysses").lower()
        return "context" if b in ("context", "cp", "ring", "allgather_kv") else "ulysses"

    def engine_model(self, engine_tp: int = 1) -> CausalLM:
        """The model object a colocated generation engine should run.  Shared with training whenever the training
        parameters are the full weights and the engine is unsharded (plain or sequence-parallel trainer); a separate
        copy in the engine's own layout otherwise (tensor-parallel trainer shards, LoRA adapters over a frozen base, a
        tensor-parallel engine) -- ``refresh_engine_model`` then brings it up to date after every update."""
        from ..models.lora import LoRACausalLM

        if getattr(self, "_engine_copy", None) is not None:
            return self._engine_copy
        if isinstance(self.model, LoRACausalLM):
            if engine_tp > 1:
                raise NotImplementedError("LoRA training with a tensor-parallel engine is not supported")
            self._engine_copy = CausalLM(self.model.args, device=self.env.device, dtype=self.model.base_flat_params.dtype,
                                         seed=None)
            self.model.merge_into(self._engine_copy)
            return self._engine_copy
        dense_tp = self._dense_tp_trainer()
        if dense_tp or (engine_tp > 1 and not self.expert_parallel and self.pipe is None):
            self._engine_copy = self._build_engine_copy(engine_tp)
            self.refresh_engine_model()
            return self._engine_copy
        if self.mesh is not None and not self.sequence_parallel:
            if engine_tp > 1:
                raise NotImplementedError("a tensor-parallel engine needs a dense data-, tensor- or sequence-parallel trainer")
            self._engine_copy = self.full_model_copy()
            return self._engine_copy
        return getattr(self, "_plain_model", None) or self.model

    def _dense_tp_trainer(self) -> bool:
        return (self.mesh is not None and not self.sequence_parallel and not self.expert_parallel and self.pipe is None)

    def _build_engine_copy(self, engine_tp: int) -> CausalLM:
        """Engine-side weights in the engine's own tensor-parallel layout, plus the block-copy plan that fills them
        from this rank's training shard (``weight_sync/relayout.py``).  With a tensor-parallel trainer the buffer is a
        symmetric allocation of the trainer's TP group, so every rank of the group can push into it."""
        from ..models.decoder import flat_numel_for
        from ..models.tp_decoder import local_args
        from ..parallel.dist import build_mesh
        from ..parallel.tensor_parallel import TPGroup
        from ..weight_sync import relayout as rlo

        dev, cuda = self.env.device, self.env.device.type == "cuda"
        dense_tp = self._dense_tp_trainer()
        src_model = self.model if dense_tp or not hasattr(self, "_plain_model") else self._plain_model
        full_args = src_model.full_args if dense_tp else src_model.args
        src_tp, src_rank = (self.mesh.tp_size, self.mesh.tp_rank) if dense_tp else (1, 0)
        dtype = src_model.flat_params.dtype
        eargs = local_args(full_args, engine_tp) if engine_tp > 1 else full_args
        numel = flat_numel_for(eargs)
        sym = None
        if dense_tp and cuda and self.tp.peer is not None:
            sym = self.tp.peer.alloc(numel, dtype)
            flat = sym.local
        else:
            flat = torch.zeros(numel, device=dev, dtype=dtype)
        if engine_tp > 1:
            from ..engine.tp_model import TPEngineModel
            from ..parallel.peer import PeerContext

            emesh = build_mesh(engine_tp, self.env)
            if cuda:
                same = dense_tp and engine_tp == src_tp
                epeer = self.tp.peer if same else PeerContext(dev, group=emesh.tp_group)
            else:
                epeer = None
            etp = TPGroup(epeer, emesh.tp_group)
            self.engine_mesh = emesh
            copy = TPEngineModel(full_args, etp, device=dev, dtype=dtype, flat_buffer=flat)
        else:
            copy = CausalLM(full_args, device=dev, dtype=dtype, seed=None, flat_buffer=flat)
        self._relayout = None
        self._relayout_src = (src_model, src_tp, src_rank, full_args, engine_tp)
        if cuda:
            base = self.env.rank - src_rank  # first global rank of this trainer TP group
            dests = [rlo.Destination(sym.ptrs[d] if sym is not None else flat.data_ptr(), copy.offsets, engine_tp,
                                     (base + d) % engine_tp) for d in range(src_tp)]
            plan = rlo.build_plan(full_args, src_model.offsets, src_tp, src_rank, dests,
                                  src_vocab_parallel_head=bool(getattr(src_model, "vocab_parallel_head", False)))
            self._relayout = rlo.RelayoutPush(plan, src_model.flat_params, dests)
        return copy

    def remote_push_plan(self, dest_ptrs: Sequence[int]):
        """Block-copy plan from this rank's training parameters into unsharded engine buffers mapped from other
        processes (``dest_ptrs``: device pointers valid in this process).  Tensor-parallel shards are re-laid out on
        the way; ranks that hold the same data (data- / sequence-parallel replicas) each push a disjoint part."""
        from ..models.decoder import param_offsets
        from ..weight_sync import relayout as rlo

        dense_tp = self._dense_tp_trainer()
        if self.expert_parallel or self.pipe is not None:
            raise NotImplementedError("peer weight push supports data-, sequence- and tensor-parallel trainers")
        src_model = self.model if dense_tp or not hasattr(self, "_plain_model") else self._plain_model
        full_args = src_model.full_args if dense_tp else src_model.args
        src_tp, src_rank = (self.mesh.tp_size, self.mesh.tp_rank) if dense_tp else (1, 0)
        reps, rep_rank = (self.mesh.dp_size, self.mesh.dp_rank) if dense_tp else (self.env.world_size, self.env.rank)
        offs = param_offsets(full_args)
        dests = [rlo.Destination(int(p), offs, 1, 0) for p in dest_ptrs]
        plan = rlo.build_plan(full_args, src_model.offsets, src_tp, src_rank, dests,
                              src_vocab_parallel_head=bool(getattr(src_model, "vocab_parallel_head", False)),
                              chunk_world=reps, chunk_rank=rep_rank)
        return rlo.RelayoutPush(plan, src_model.flat_params, dests)

    def refresh_engine_model(self) -> None:
        """Bring a separate engine copy up to date with the trained parameters (no-op when the buffer is shared)."""
        from ..models.lora import LoRACausalLM

        ec = getattr(self, "_engine_copy", None)
        if ec is None:
            return
        if isinstance(self.model, LoRACausalLM):
            self.model.merge_into(ec)
            return
        if getattr(self, "_relayout_src", None) is None:
            self.full_model_copy(into=ec)
            return
        src_model, src_tp, src_rank, full_args, engine_tp = self._relayout_src
        if getattr(self, "_relayout", None) is not None:
            # one kernel: every block this rank owns goes straight into the engine buffers that need it (peer stores);
            # the barrier makes every rank's pushes visible before any engine of the group reads its weights
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            self._relayout.run()
            if src_tp > 1:
                self.tp.peer.barrier(3)
            ev1.record()
            ev1.synchronize()
            self.last_weight_sync_ms = ev0.elapsed_time(ev1)
            self.last_weight_sync_bytes = self._relayout.bytes_out
            return
        # host / gloo path: gather the full state, then slice it the way the engine shards it
        from ..models.tp_decoder import shard_param

        state = src_model.gather_full_state() if src_tp > 1 else dict(src_model.named_flat_views())
        erank = self.env.rank % engine_tp
        with torch.no_grad():
            for name, prm in ec.named_flat_views():
                prm.copy_(shard_param(name, state[name].detach(), full_args, engine_tp, erank) if engine_tp > 1
                          else state[name])

    @staticmethod
    def _ep_size_from_cfg(cfg) -> int:
        if getattr(cfg, "strategy", "fsdp") != "megatron":
            return 1
        return int(getattr(cfg.policy.megatron_config, "expert_model_parallel_size", 1) or 1)

    @staticmethod
    def _pp_size_from_cfg(cfg) -> int:
        if getattr(cfg, "strategy", "fsdp") != "megatron":
            return 1
        return int(getattr(cfg.policy.megatron_config, "pipeline_model_parallel_size", 1) or 1)

    @staticmethod
    def _tp_size_from_cfg(cfg) -> int:
        if getattr(cfg, "strategy", "fsdp") != "megatron":
            return 1
        return int(getattr(cfg.policy.megatron_config, "tensor_model_parallel_size", 1) or 1)

    def full_model_copy(self, into: Optional[CausalLM] = None) -> CausalLM:
        """Unsharded copy of a tensor-parallel model (collective over the TP group); ``into`` is updated in place."""
        if into is None:
            into = CausalLM(self.model.full_args, device=self.env.device, dtype=self.model.flat_params.dtype, seed=None)
        with torch.no_grad():
            if hasattr(self.model, "iter_full_state"):
                for name, full in self.model.iter_full_state():  # one parameter in flight at a time
                    into.p(name).copy_(full)
            else:
                state = self.model.gather_full_state()
                for name, prm in into.named_flat_views():
                    prm.copy_(state[name])
        return into

    @property
    def tp_size(self) -> int:
        """Ranks that jointly process one data shard (tensor- or sequence-parallel group size; expert-parallel ranks
        each keep their own data)."""
        return self.mesh.tp_size if (self.mesh is not None and not getattr(self, "expert_parallel", False)) else 1

    def _pipe_begin_all(self, batch: TrainingInputBatch, groups, n_mb: int, temp: float, with_entropy: bool = False):
        """Pipeline parallelism: pack every micro-batch and start it through the stages before any result is collected,
        so that stage ``s`` works on micro-batch ``k`` while stage ``s - 1`` works on ``k + 1``.  Returns the
        ``(rows, packed view, handle)`` triples the loops finish with ``self.pipe.pred_logprobs_end``."""
        started = []
        for k in range(n_mb):
            rows = groups[k] if k < len(groups) else groups[-1]
            pv = self._pack(batch, rows)
            started.append((rows, pv, self.pipe.pred_logprobs_begin(pv.ids, pv.positions, pv.cu_seqlens, pv.max_seqlen,
                                                                    pv.pred_index, pv.targets, temp, with_entropy)))
        return started

    def _pred_logprobs(self, pv: PackedView, temp: float, with_entropy: bool = False):
        """Log-probs (and entropies) of the packed batch's prediction positions, ``[n_pred]`` each."""
        if self.mesh is None:
            h = self._hidden(pv)
            return self.model.token_logprobs(h[pv.pred_index], pv.targets, temp, with_entropy=with_entropy)
        from ..models.tp_decoder import pad_packed_for_tp

        if self.pipe is not None:
            return self.pipe.pred_logprobs(pv.ids, pv.positions, pv.cu_seqlens, pv.max_seqlen, pv.pred_index, pv.targets,
                                           temp, with_entropy=with_entropy)
        if self.expert_parallel:
            # every rank routes its own tokens, but the routing tables are exchanged as equal-sized blocks: pad this
            # rank's packed batch to the longest one in the expert-parallel group
            T = pv.ids.numel()
            tmax = torch.tensor([T], device=pv.ids.device, dtype=torch.int64)
            if dist.is_initialized() and self.mesh.tp_size > 1:
                dist.all_reduce(tmax, op=dist.ReduceOp.MAX, group=self.mesh.tp_group)
            target = (int(tmax) + 7) // 8 * 8
            ids, pos, cu = pv.ids, pv.positions, pv.cu_seqlens
            if target > T:
                n = target - T
                ids = torch.cat([ids, torch.zeros(n, dtype=ids.dtype, device=ids.device)])
                pos = torch.cat([pos, torch.arange(n, dtype=pos.dtype, device=pos.device)])
                cu = torch.cat([cu, torch.tensor([target], dtype=cu.dtype, device=cu.device)])
            if pv.routing is not None or self._replay_on:
                from ..models import router_replay

                r = pv.routing
                if r is not None and target > T:
                    r = torch.cat([r, r.new_full((target - T, *r.shape[1:]), -1)], 0)
                router_replay.set_replay(r)
                self._replay_on = r is not None
            h = self.model(ids, pos, cu, max(pv.max_seqlen, target - T))
            return self.model.token_logprobs(h[pv.pred_index], pv.targets, temp, with_entropy=with_entropy)

        ids, pos, cu, T = pad_packed_for_tp(pv.ids, pv.positions, pv.cu_seqlens, self.mesh.tp_size)
        h = self.model(ids, pos, cu, max(pv.max_seqlen, ids.numel() - T))
        tgt = torch.zeros(ids.numel(), dtype=pv.targets.dtype, device=ids.device)
        tgt[pv.pred_index] = pv.targets
        lp, ent = self.model.token_logprobs_full(h, tgt, temp, with_entropy=with_entropy)
        return lp[pv.pred_index], (ent[pv.pred_index] if ent is not None else None)

    def _pred_values(self, pv: PackedView) -> torch.Tensor:
        """Value-head outputs at the packed batch's prediction positions, ``[n_pred]``."""
        if self.mesh is None:
            return self.model.values(self._hidden(pv)[pv.pred_index])
        if self.pipe is not None or self.expert_parallel:
            raise NotImplementedError("the critic supports data, tensor and sequence parallelism")
        from ..models.tp_decoder import pad_packed_for_tp

        ids, pos, cu, T = pad_packed_for_tp(pv.ids, pv.positions, pv.cu_seqlens, self.mesh.tp_size)
        h = self.model(ids, pos, cu, max(pv.max_seqlen, ids.numel() - T))
        return self.model.values_full(h)[pv.pred_index]

    # ------------------------------------------------------------------ forward (no grad)
    @torch.no_grad()
    def forward(self, batch: TrainingInputBatch, train_packing: bool = False) -> TrainingOutputBatch:
        """Log-probabilities (policy/ref) or values (critic) on the right-aligned response grid ``[B, R]``.

        ``train_packing`` groups the rows exactly as ``forward_backward`` will (``micro_train_batch_size_per_gpu``), so
        that the values a later training pass recomputes for the same mini-batch come from identically packed
        micro-batches (``trainer.recompute_old_logprobs_per_minibatch``, reference: trainer.py:1244-1277)."""
        self.backload()
        B, R = batch["response_mask"].shape
        out = torch.zeros((B, R), dtype=torch.float32)
        mbs = self.cfg.micro_train_batch_size_per_gpu if train_packing else self.cfg.micro_forward_batch_size_per_gpu
        groups = microbatch_indices(self._seq_lens(batch), mbs, self._max_tokens(),
                                    getattr(self.cfg.b200, "microbatch_packing", "balanced"))
        n_mb = self._num_microbatches(len(groups))
        temp = float(self.cfg.algorithm.temperature or 1.0)
        was_ckpt = self.model.gradient_checkpointing
        self.model.gradient_checkpointing = False
        started = self._pipe_begin_all(batch, groups, n_mb, temp) if (self.pipe is not None and self.role != "critic") else None
        for k in range(n_mb):
            rows = groups[k] if k < len(groups) else groups[-1]  # padding micro-batch keeps collectives aligned
            if started is not None:
                _, pv, handle = started[k]
                started[k] = None
                vals = self.pipe.pred_logprobs_end(handle)[0]
                if k < len(groups):
                    out[torch.tensor(rows, dtype=torch.long)] = _lib.to_host(pv.scatter_to_grid(vals.float()))
                continue
            pv = self._pack(batch, rows)
            if self.role == "critic":
                if pv.pred_index.numel() == 0 and self.mesh is None:
                    continue
                vals = self._pred_values(pv)
            else:
                if pv.pred_index.numel() == 0 and self.mesh is None:
                    self._hidden(pv)
                    continue
                vals = self._pred_logprobs(pv, temp)[0]
            if k < len(groups):
                grid = _lib.to_host(pv.scatter_to_grid(vals.float()))
                out[torch.tensor(rows, dtype=torch.long)] = grid
        self.model.gradient_checkpointing = was_ckpt
        self._end_replay()
        return TrainingOutputBatch({"output": out})

    # ------------------------------------------------------------------ state movement (colocation)
    def offload(self, include_optimizer: bool = True, include_params: bool = True) -> None:
        """Move parameters / optimizer state to pinned host memory (colocated GPU sharing)."""
        if self.env.device.type != "cuda":
            return
        if include_optimizer and self.optimizer is not None:
            self.optimizer.offload()
        if include_params and self._on_device and not self.trainable:
            host = torch.empty(self.model.flat_params.shape, dtype=self.model.flat_params.dtype, pin_memory=True)
            host.copy_(self.model.flat_params)
            self._offloaded["params"] = host
            # keep the storage object (views must stay valid): shrink it to zero bytes
            self.model.flat_params.untyped_storage().resize_(0)
            self._on_device = False
        torch.cuda.empty_cache()

    def backload(self, include_optimizer: bool = True) -> None:
        if self.env.device.type != "cuda":
            return
        if not self._on_device:
            host = self._offloaded.pop("params")
            st = self.model.flat_params.untyped_storage()
            st.resize_(host.numel() * host.element_size())
            self.model.flat_params.copy_(host, non_blocking=True)
            self._on_device = True
        if include_optimizer and self.optimizer is not None:
            self.optimizer.backload()

    # ------------------------------------------------------------------ optimizer
    def optim_step(self) -> Optional[float]:
        """Reduce gradients across ranks, clip, AdamW, LR schedule, zero grads. Returns the gradient norm."""
        assert self.optimizer is not None
        self.backload()
        scale = 1.0
        if self.role == "critic" and self.num_microbatches_accumulated > 0:
            scale = 1.0 / self.num_microbatches_accumulated  # reference: worker.py:1513-1537
        if self.mesh is not None:
            self.model.reduce_replicated_grads()
        frozen = self._frozen_ranges()
        kept = []
        if frozen:
            # frozen parameters: no gradient (so they do not count in the clipping norm either) and, because AdamW's
            # weight decay would still shrink them, their values -- working copy and fp32 master -- put back afterwards
            o = self.optimizer
            for lo, hi in frozen:
                self.flat_grad[lo:hi].zero_()
                m0, m1 = max(lo, o.lo), min(hi, o.lo + o.shard)
                kept.append((lo, hi, self.model.flat_params[lo:hi].clone(), m0, m1,
                             o.master[m0 - o.lo : m1 - o.lo].clone() if m1 > m0 else None))
        norm = self.optimizer.step(grad_scale=scale)
        for lo, hi, p, m0, m1, mast in kept:
            self.model.flat_params[lo:hi].copy_(p)
            if mast is not None:
                self.optimizer.master[m0 - self.optimizer.lo : m1 - self.optimizer.lo].copy_(mast)
        # the fused optimizer publishes nothing once the status word is set (csrc/comm.cu); tell the caller
        self.check_device_status("optim_step")
        self.scheduler.step()
        self.optimizer.zero_grad()
        self.num_microbatches_accumulated = 0
        return norm

    def _frozen_ranges(self) -> List[Tuple[int, int]]:
        """Flat-buffer ranges that training must not move: the routers of a mixture-of-experts policy under
        ``megatron_config.freeze_moe_router`` (reference: megatron_worker.py, same key)."""
        if getattr(self, "_frozen_cache", None) is not None:
            return self._frozen_cache
        out: List[Tuple[int, int]] = []
        node = getattr(self.cfg, self.role, None) if self.role in ("policy", "critic") else None
        if (node is not None and getattr(getattr(node, "megatron_config", None), "freeze_moe_router", False)
                and getattr(self.model.args, "num_experts", 0) and hasattr(self.model, "offsets")):
            for name, (off, n) in self.model.offsets.items():
                if name.endswith(".router"):
                    out.append((off, off + n))
        self._frozen_cache = out
        return out

    def set_lr(self, lr: float) -> None:
        self.optimizer.set_lr(lr)

    def get_lr(self) -> float:
        return self.optimizer.lr

    # ------------------------------------------------------------------ checkpoints (FSDP-style per-rank layout)
    def save_checkpoint(self, ckpt_dir: str, tag: Optional[str] = None, client_state: Optional[dict] = None) -> None:
        """Per-rank files ``{model,optim,extra_state}_world_size_{W}_rank_{r}.pt`` (+ ``huggingface/`` on rank 0).

        File naming follows the reference layout (fsdp_strategy.py:391-444); the model file holds this rank's
        contiguous slice of the flat parameter buffer instead of pickled DTensors.
        """
        os.makedirs(ckpt_dir, exist_ok=True)
        W, r = self.env.world_size, self.env.rank
        n = self.model.flat_params.numel()
        # with tensor parallelism each TP rank owns a different buffer, sliced over its data-parallel peers
        dp = self.mesh.dp_size if self.mesh is not None else W
        dpr = self.mesh.dp_rank if self.mesh is not None else r
        shard = n // dp
        lo = dpr * shard
        torch.save({"flat_shard": self.model.flat_params[lo : lo + shard].cpu(), "offset": lo, "numel": n,
                    "specs": self.model.specs, "tp_size": self.tp_size,
                    "tp_rank": self.mesh.tp_rank if self.mesh is not None else 0},
                   os.path.join(ckpt_dir, f"model_world_size_{W}_rank_{r}.pt"))
        if self.optimizer is not None:
            sd = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in self.optimizer.state_dict().items()}
            torch.save(sd, os.path.join(ckpt_dir, f"optim_world_size_{W}_rank_{r}.pt"))
        extra = {"lr_scheduler": self.scheduler.state_dict() if self.scheduler else None, "client_state": client_state or {},
                 "tag": tag, "fsdp_strategy": "flat_zero", "world_size": W, "rank": r,
                 "rng": {"torch": torch.get_rng_state(), "numpy": np.random.get_state(),
                         "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}}
        torch.save(extra, os.path.join(ckpt_dir, f"extra_state_world_size_{W}_rank_{r}.pt"))
        if r == 0 and hasattr(self.model, "save_adapter"):
            self.model.save_adapter(os.path.join(ckpt_dir, "lora_adapter"))  # PEFT layout, as the reference writes
        if r == 0:
            import json

            hf_dir = os.path.join(ckpt_dir, "huggingface")
            os.makedirs(hf_dir, exist_ok=True)
            with open(os.path.join(hf_dir, "config.json"), "w") as f:
                json.dump(self.model.args.to_hf_config(), f, indent=1)
            with open(os.path.join(ckpt_dir, "fsdp_config.json"), "w") as f:
                json.dump({"FSDP_version": 2, "world_size": W, "layout": "flat_zero", "tensor_parallel_size": self.tp_size}, f)
        if dist.is_initialized():
            dist.barrier()

    def load_checkpoint(self, ckpt_dir: str, load_optimizer_states: bool = True, load_lr_scheduler_states: bool = True):
        W, r = self.env.world_size, self.env.rank
        path = os.path.join(ckpt_dir, f"model_world_size_{W}_rank_{r}.pt")
        if not os.path.exists(path):
            have = sorted(f for f in os.listdir(ckpt_dir) if f.startswith("model_world_size_"))
            raise FileNotFoundError(f"{path} not found (checkpoint was written for a different world size? found: {have})")
        n = self.model.flat_params.numel()
        # every rank needs its full parameter buffer: read the slices of all ranks that share it
        tp = self.tp_size
        for rr in (range(W) if self.mesh is None else range(self.mesh.tp_rank, W, tp)):
            d = torch.load(os.path.join(ckpt_dir, f"model_world_size_{W}_rank_{rr}.pt"), weights_only=False)
            assert d["numel"] == n, "checkpoint parameter layout differs from the model"
            self.model.flat_params[d["offset"] : d["offset"] + d["flat_shard"].numel()].copy_(d["flat_shard"])
        if self.optimizer is not None and load_optimizer_states:
            sd = torch.load(os.path.join(ckpt_dir, f"optim_world_size_{W}_rank_{r}.pt"), weights_only=False)
            self.optimizer.load_state_dict(sd)
        extra = torch.load(os.path.join(ckpt_dir, f"extra_state_world_size_{W}_rank_{r}.pt"), weights_only=False)
        if self.scheduler is not None and load_lr_scheduler_states and extra.get("lr_scheduler"):
            self.scheduler.load_state_dict(extra["lr_scheduler"])
        rng = extra.get("rng") or {}
        if rng.get("torch") is not None:
            torch.set_rng_state(rng["torch"])
        if rng.get("numpy") is not None:
            np.random.set_state(rng["numpy"])
        if rng.get("cuda") is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(rng["cuda"])
        return ckpt_dir, extra.get("client_state", {})

    def save_hf_model(self, export_dir: str, tokenizer=None) -> None:
        from ..models import hf_io

        from ..models.lora import LoRACausalLM

        model = self.model
        if isinstance(model, LoRACausalLM):  # merged weights + the adapter itself
            if self.env.rank == 0:
                model.save_adapter(os.path.join(export_dir, "lora_adapter"))
            merged = CausalLM(model.args, device=self.env.device, dtype=model.base_flat_params.dtype, seed=None)
            model.merge_into(merged)
            model = merged
        elif self.mesh is not None and not self.sequence_parallel:  # gather the TP shards for the export
            model = self.full_model_copy()
        if self.env.rank == 0:
            hf_io.save_hf_model(model, export_dir, tokenizer)
        if dist.is_initialized():
            dist.barrier()


class RefWorker(ModelWorker):
    role = "ref"

    def __init__(self, cfg, **kw):
        super().__init__(cfg, trainable=False, **kw)


class PolicyWorker(ModelWorker):
    role = "policy"

    def __init__(self, cfg, **kw):
        super().__init__(cfg, trainable=True, optimizer_cfg=cfg.policy.optimizer_config, **kw)
        self.mtp_head = self.mtp_optimizer = None
        mcfg = getattr(cfg, "mtp", None)
        if mcfg is not None and mcfg.enabled:
            # Draft head for speculative decoding, trained beside the policy on detached trunk states with its own
            # optimizer and its own gradient clipping (reference: skyrl/backends/skyrl_train/mtp/*, trainer.mtp).
            if self.mesh is not None:
                raise NotImplementedError("trainer.mtp.enabled is supported with the data-parallel strategy only")
            from ..algorithms.mtp import DraftHead

            torch.manual_seed(int(getattr(cfg, "seed", 0)) + 7919)  # identical initial head on every rank
            self.mtp_head = DraftHead(self.model.args.hidden_size, dtype=torch.float32, device=self.env.device)
            ocfg = cfg.policy.optimizer_config
            self.mtp_optimizer = torch.optim.AdamW(self.mtp_head.parameters(), lr=ocfg.lr, betas=tuple(ocfg.adam_betas),
                                                   weight_decay=ocfg.weight_decay)
            self._mtp_loss_sum, self._mtp_loss_n = 0.0, 0

    def _hidden(self, pv):
        h = super()._hidden(pv)
        if self.mtp_head is not None and torch.is_grad_enabled():
            self._mtp_hidden = h.detach()
        return h

    def _mtp_accumulate(self, pv, mask_pred: torch.Tensor, n_mb: int) -> None:
        """Draft-head loss of one micro-batch on the trunk states its policy forward just produced."""
        from ..algorithms.mtp import mtp_draft_backward

        h = getattr(self, "_mtp_hidden", None)
        if h is None:
            return
        tok_mask = torch.zeros(h.shape[0], dtype=torch.bool, device=h.device)
        tok_mask[pv.pred_index] = mask_pred > 0
        loss = mtp_draft_backward(self.mtp_head, h, self.model.lm_head_weight(), pv.cu_seqlens, tok_mask,
                                  float(self.cfg.algorithm.temperature or 1.0),
                                  scale=float(self.cfg.mtp.loss_weight) / max(1, n_mb))
        self._mtp_loss_sum += float(loss)
        self._mtp_loss_n += 1
        self._mtp_hidden = None

    def optim_step(self):
        norm = super().optim_step()
        if self.mtp_head is not None:
            from ..algorithms.mtp import clip_grad_norm_separately

            params = [p for p in self.mtp_head.parameters() if p.grad is not None]
            W = self.env.world_size
            if W > 1 and dist.is_initialized():
                for p in params:
                    dist.all_reduce(p.grad)
                    p.grad.div_(W)
            gn, _ = clip_grad_norm_separately(params, float(self.cfg.policy.optimizer_config.max_grad_norm or 1.0))
            self.mtp_optimizer.step()
            self.mtp_optimizer.zero_grad(set_to_none=True)
            self.last_mtp = {"mtp_loss": self._mtp_loss_sum / max(1, self._mtp_loss_n), "mtp_grad_norm": gn}
            self._mtp_loss_sum, self._mtp_loss_n = 0.0, 0
        return norm

    def save_checkpoint(self, ckpt_dir: str, tag: Optional[str] = None, client_state: Optional[dict] = None) -> None:
        super().save_checkpoint(ckpt_dir, tag, client_state)
        if self.mtp_head is not None and self.env.is_main:  # the head is replicated: one copy is enough
            torch.save({"head": self.mtp_head.state_dict(), "optim": self.mtp_optimizer.state_dict()},
                       os.path.join(ckpt_dir, "mtp_head.pt"))

    def load_checkpoint(self, ckpt_dir: str, *a, **kw):
        out = super().load_checkpoint(ckpt_dir, *a, **kw)
        path = os.path.join(ckpt_dir, "mtp_head.pt")
        if self.mtp_head is not None and os.path.exists(path):
            st = torch.load(path, map_location=self.env.device, weights_only=False)
            self.mtp_head.load_state_dict(st["head"])
            self.mtp_optimizer.load_state_dict(st["optim"])
        return out

    def _layer_buckets(self) -> List[Tuple[int, int]]:
        """Flat gradient range of every decoder layer; the last layer's range also covers the final norm and head."""
        m = self.model
        L = m.args.num_layers
        starts = [m.offsets[f"layers.{i}.ln1"][0] for i in range(L)]
        ends = starts[1:] + [m.flat_params.numel()]
        return list(zip(starts, ends))

    def forward_backward(self, batch: TrainingInputBatch, loss_fn: Optional[str] = None,
                         loss_fn_config: Optional[dict] = None, return_per_token_outputs: bool = False,
                         step_follows: bool = False) -> Dict[str, Any]:
        """One mini-batch: micro-batch loop accumulating gradients. Advantages must already be reduction-scaled.

        ``step_follows``: the caller runs ``optim_step`` right after this call, so the gradients of a layer are final
        as soon as the *last* micro-batch's backward pass has left that layer; with the fused peer optimizer their
        reduce-scatter then starts behind the backward pass, layer by layer (reference behaviour: FSDP2 reduce-scatters
        each layer's gradients inside backward, fsdp_utils.py:209-235)."""
        self.backload()
        algo = self.cfg.algorithm
        if loss_fn_config:
            import copy

            algo = copy.deepcopy(algo)
            for k, v in loss_fn_config.items():
                if not hasattr(algo, k):
                    raise ValueError(f"loss_fn_config: the algorithm config has no field '{k}'")
                if isinstance(v, dict):  # nested section (dppo, cispo, sapo ...): set its fields
                    node = getattr(algo, k)
                    for kk, vv in v.items():
                        if not hasattr(node, kk):
                            raise ValueError(f"loss_fn_config: '{k}' has no field '{kk}'")
                        setattr(node, kk, vv)
                else:
                    setattr(algo, k, v)
        loss_name = loss_fn or algo.policy_loss_type
        loss_name = {"ppo": "regular"}.get(loss_name, loss_name)
        if loss_name != algo.policy_loss_type:
            import copy

            algo = copy.deepcopy(algo)
            algo.policy_loss_type = loss_name
        loss_func = rl.PolicyLossRegistry.get(loss_name)
        dev = self.env.device
        B, R = batch["response_mask"].shape
        groups = microbatch_indices(self._seq_lens(batch), self.cfg.micro_train_batch_size_per_gpu, self._max_tokens(),
                                    getattr(self.cfg.b200, "microbatch_packing", "balanced"))
        n_mb = self._num_microbatches(len(groups))
        # number of distinct data shards (expert-parallel ranks each hold their own)
        world = self.mesh.dp_size if (self.mesh is not None and not self.expert_parallel) else self.env.world_size
        temp = float(algo.temperature or 1.0)
        use_kl = bool(algo.use_kl_loss) and batch.get("base_action_log_probs") is not None and loss_name != "cross_entropy"
        use_ent = bool(algo.use_entropy_loss) and loss_name != "cross_entropy"
        fused = dev.type == "cuda" and rl.fused_objective_supported(algo) and loss_name in ("regular", "dual_clip") \
            and not return_per_token_outputs
        all_metrics: List[Dict[str, float]] = []
        per_row_logprobs = torch.zeros((B, R), dtype=torch.float32) if return_per_token_outputs else None
        overlap = (step_follows and self.mesh is None and type(self.model) is CausalLM and self.optimizer is not None
                   and self.optimizer.can_overlap_reduce and getattr(self.cfg.b200, "overlap_grad_reduce", True))
        # pipeline parallelism: all forwards first, then loss + backward per micro-batch (activations of a stage stay
        # alive for all micro-batches, which gradient checkpointing keeps to the layer inputs)
        started = self._pipe_begin_all(batch, groups, n_mb, temp, use_ent) if self.pipe is not None else None
        for k in range(n_mb):
            real = k < len(groups)
            rows = groups[k] if real else groups[-1]
            if started is not None:
                _, pv, handle = started[k]
                started[k] = None
                lp, ent = self.pipe.pred_logprobs_end(handle)
            else:
                pv = self._pack(batch, rows)
                if overlap and k == n_mb - 1:
                    buckets = self._layer_buckets()
                    self.model.layer_grads_ready = lambda i, b=buckets: self.optimizer.reduce_bucket(*b[i])
                lp, ent = self._pred_logprobs(pv, temp, with_entropy=use_ent)
            weight = len(rows) / max(1, B * world)  # KL / entropy terms: mean over the global mini-batch
            g = lambda key: self._rows_to_device(batch.get(key), rows)  # noqa: E731
            mask_g, adv_g = g("loss_mask"), g("advantages")
            old_g, ref_g, roll_g = g("action_log_probs"), g("base_action_log_probs"), g("rollout_logprobs")
            if old_g is None:
                old_g = pv.scatter_to_grid(lp.detach().float())
            m: Dict[str, float] = {}
            if fused:
                mask_f = pv.gather_from_grid(mask_g)
                klw = None
                if use_kl:
                    per_seq = mask_g.sum(-1, keepdim=True).clamp(min=1.0) * len(rows)
                    klw = pv.gather_from_grid((1.0 / per_seq).expand_as(mask_g))
                total, stats = rl.FusedPolicyObjective.apply(
                    lp.float(), pv.gather_from_grid(old_g), pv.gather_from_grid(adv_g), mask_f,
                    pv.gather_from_grid(ref_g) if use_kl else None, None, klw, algo.eps_clip_low, algo.eps_clip_high,
                    algo.clip_ratio_c, loss_name == "dual_clip", algo.kl_estimator_type, 1.0,
                    algo.kl_loss_coef * weight if use_kl else 0.0)
                loss = total
                entropy_mean = None
                if ent is not None:
                    entropy_mean = (ent.float() * mask_f).sum() / mask_f.sum().clamp(min=1.0)
                    if use_ent:
                        loss = loss - algo.entropy_loss_coef * weight * entropy_mean
                st = stats.detach()
                m.update(policy_loss=st[0], policy_kl=st[2] if use_kl else 0.0,
                         **{"loss_metrics/clip_ratio": st[1] / st[3].clamp(min=1.0)})
                if entropy_mean is not None:
                    m["policy_entropy"] = entropy_mean.detach()
            else:
                lp_grid = pv.scatter_to_grid(lp.float())
                policy_loss, lm = loss_func(lp_grid, old_g, adv_g if adv_g is not None else torch.zeros_like(lp_grid),
                                            algo, loss_mask=mask_g, rollout_logprobs=roll_g)
                loss = policy_loss
                m["policy_loss"] = policy_loss.detach()
                m.update({"loss_metrics/" + kk: float(vv) for kk, vv in lm.items()})
                if loss_name != "cross_entropy":
                    if ent is not None:
                        ent_grid = pv.scatter_to_grid(ent.float())
                        entropy_mean = masked_mean(ent_grid, mask_g)
                        m["policy_entropy"] = entropy_mean.detach()
                        if use_ent:
                            loss = loss - algo.entropy_loss_coef * weight * entropy_mean
                    if use_kl:
                        kl = rl.compute_approx_kl(lp_grid, ref_g, loss_mask=mask_g, kl_estimator_type=algo.kl_estimator_type)
                        kl_mean = masked_mean(kl, mask_g, dim=-1).mean()
                        loss = loss + algo.kl_loss_coef * weight * kl_mean
                        m["policy_kl"] = kl_mean.detach()
                if per_row_logprobs is not None and real:
                    per_row_logprobs[torch.tensor(rows, dtype=torch.long)] = lp_grid.detach().cpu()
            if not real:
                loss = loss * 0.0
            loss.backward()
            self.model.layer_grads_ready = None
            if real and self.mtp_head is not None:
                self._mtp_accumulate(pv, pv.gather_from_grid(mask_g), n_mb)
            if real:
                m["final_loss"] = loss.detach()
                if roll_g is not None:
                    d = (pv.scatter_to_grid(lp.detach().float()) - roll_g).abs()
                    m["rollout_train_logprobs_abs_diff_mean"] = masked_mean(d, mask_g)
                all_metrics.append(m)
            self.num_microbatches_accumulated += 1
        self._end_replay()
        status = reduce_metrics(materialize_metrics(all_metrics))
        status = all_reduce_metrics(status, self.env)
        status["policy_lr"] = self.optimizer.lr
        status["response_length"] = R
        if self.mtp_head is not None and self._mtp_loss_n:
            status["mtp_loss"] = self._mtp_loss_sum / self._mtp_loss_n
        if per_row_logprobs is not None:
            rm = batch["response_mask"]
            lm_ = batch.get("loss_mask")
            outs = []
            for i in range(B):
                n = int(rm[i].sum())
                row = per_row_logprobs[i, R - n:].tolist() if n else []
                o = {"logprobs": row}
                if loss_name == "cross_entropy":
                    w = lm_[i, R - n:].tolist() if (lm_ is not None and n) else [1.0] * n
                    o["elementwise_loss"] = [-a * b for a, b in zip(row, w)]
                outs.append(o)
            status["loss_fn_outputs"] = outs
        return status


class CriticWorker(ModelWorker):
    role = "critic"

    def __init__(self, cfg, **kw):
        super().__init__(cfg, trainable=True, value_head=True, optimizer_cfg=cfg.critic.optimizer_config, **kw)

    def forward_backward(self, batch: TrainingInputBatch, **_unused) -> Dict[str, Any]:
        """Clipped value loss over the mini-batch; gradients are averaged over micro-batches at ``optim_step``."""
        self.backload()
        algo = self.cfg.algorithm
        B, R = batch["response_mask"].shape
        groups = microbatch_indices(self._seq_lens(batch), self.cfg.micro_train_batch_size_per_gpu, self._max_tokens(),
                                    getattr(self.cfg.b200, "microbatch_packing", "balanced"))
        n_mb = self._num_microbatches(len(groups))
        all_metrics = []
        for k in range(n_mb):
            real = k < len(groups)
            rows = groups[k] if real else groups[-1]
            pv = self._pack(batch, rows)
            v = self._pred_values(pv)
            v_grid = pv.scatter_to_grid(v)
            g = lambda key: self._rows_to_device(batch.get(key), rows)  # noqa: E731
            loss, clipfrac = rl.ppo_critic_loss(v_grid, g("values"), g("returns"), algo, loss_mask=g("loss_mask"))
            if not real:
                loss = loss * 0.0
            # mean over the data shards: ranks of one tensor / sequence parallel group hold the same shard
            (loss / max(1, self.env.world_size // self.tp_size)).backward()
            if real:
                mk = g("loss_mask")
                all_metrics.append({"critic_loss": loss.detach(), "values_mean": masked_mean(v_grid.detach(), mk),
                                    "values_clipfrac": float(clipfrac or 0.0)})
            self.num_microbatches_accumulated += 1
        st = reduce_metrics(materialize_metrics(all_metrics))
        if "critic_loss" in st and all_metrics:
            st["critic_loss"] = st["critic_loss"] / len(all_metrics)
        st = all_reduce_metrics(st, self.env)
        st["critic_lr"] = self.optimizer.lr
        return st
