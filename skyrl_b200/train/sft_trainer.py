"""Supervised fine-tuning on the same workers, kernels and sharded optimizer as RL training.

Reference: skyrl/train/sft_trainer.py:794-2258 (``SFTTrainer.setup/train/train_step/run_eval/save_checkpoint``).
One step = collate ``batch_size`` examples (padded, or grouped into FFD bins) -> every rank takes its contiguous
share -> ``PolicyWorker.forward_backward(loss_fn="cross_entropy")`` over token-budget micro-batches ->
``optim_step``.  The loss is the mean negative log-likelihood per trained token of the *global* batch: the loss
mask is divided by the global trained-token count before the (summing) loss and the (summing) gradient reduction.
"""

from __future__ import annotations

import math
import os
import time
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..config.config import TrainerConfig
from ..config.sft_config import SFTConfig
from ..parallel.dist import DistEnv, get_env
from ..workers.worker import PolicyWorker
from . import sft_data
from . import utils as tutils
from .batch import TrainingInputBatch
from .callbacks import CallbackHandler, TrainingCallback
from .tracking import Tracking


def _worker_cfg(c: SFTConfig) -> TrainerConfig:
    """The worker reads a trainer config; fill it from the SFT config."""
    t = TrainerConfig()
    t.policy.model = c.model
    t.policy.optimizer_config = c.optimizer_config
    t.policy.fsdp_config = c.fsdp_config
    t.policy.sequence_parallel_size = c.sequence_parallel_size
    t.strategy = c.strategy
    t.bf16 = c.bf16
    t.seed = c.seed
    t.gradient_checkpointing = c.gradient_checkpointing
    t.micro_train_batch_size_per_gpu = c.micro_train_batch_size_per_gpu
    t.micro_forward_batch_size_per_gpu = c.micro_train_batch_size_per_gpu
    t.max_tokens_per_microbatch = c.max_tokens_per_microbatch or -1
    t.remove_microbatch_padding = c.remove_microbatch_padding
    t.algorithm.policy_loss_type = "cross_entropy"
    t.algorithm.use_kl_loss = False
    t.algorithm.use_entropy_loss = False
    t.algorithm.temperature = 1.0
    return t


class SFTTrainer:
    def __init__(self, cfg: SFTConfig, tokenizer=None, env: Optional[DistEnv] = None, model=None,
                 train_examples: Optional[List[dict]] = None, eval_examples: Optional[List[Tuple[str, List[dict]]]] = None):
        self.cfg = cfg
        self.env = env or get_env()
        self.tokenizer = tokenizer
        self._model = model
        self.train_examples = train_examples
        self.eval_examples = eval_examples
        self.policy: Optional[PolicyWorker] = None
        self.tracker: Optional[Tracking] = None
        self.callbacks = CallbackHandler([])
        self.sampler: Optional[sft_data.StatefulSampler] = None
        self.collator = None
        self.global_step = 0
        self._validate()

    # ------------------------------------------------------------------ set-up
    def _validate(self) -> None:
        c, W = self.cfg, self.env.world_size
        if not c.use_sequence_packing and c.batch_size % W != 0:
            raise ValueError(f"batch_size={c.batch_size} must be divisible by the number of ranks ({W})")
        expect = c.placement.num_nodes * c.placement.num_gpus_per_node
        if expect != W and expect != 1:
            raise ValueError(f"placement asks for {expect} GPUs but {W} ranks were launched")

    def add_callback(self, cb: TrainingCallback) -> None:
        self.callbacks.add(cb)

    def setup(self) -> "SFTTrainer":
        c = self.cfg
        if self.tokenizer is None:
            from ..models.decoder import PRESETS
            from ..utils.tokenizer import get_tokenizer

            vocab = PRESETS[c.model.path].vocab_size if c.model.path in PRESETS else None
            self.tokenizer = get_tokenizer(c.model.path, vocab_size=vocab)
        self.policy = PolicyWorker(_worker_cfg(c), model=self._model, model_path=c.model.path, env=self.env, seed=c.seed)
        if self.env.is_main:
            self.tracker = Tracking(c.project_name, c.run_name, c.logger, config=c.to_dict(), log_dir=c.log_path, tags=c.tags)
        if c.use_sequence_packing:
            cap = c.max_tokens_per_microbatch or c.max_length
            self.collator = sft_data.PackedDataCollator(self.tokenizer, cap, dp_size=self.env.world_size)
        else:
            self.collator = sft_data.DefaultCollator(self.tokenizer, c.micro_train_batch_size_per_gpu)
        return self

    def load_dataset(self) -> List[dict]:
        if self.train_examples is not None:
            return self.train_examples
        c = self.cfg
        ex: List[dict] = []
        self._source_sizes: List[int] = []
        for p in (c.pretokenized_dataset_paths or []):
            rows = sft_data.load_pretokenized(p)
            ex.extend(rows)
            self._source_sizes.append(len(rows))
        for i, src in enumerate(c.train_sources()):
            split = (c.train_dataset_splits or [c.dataset_split] * (i + 1))[i] if (c.train_dataset_splits or c.dataset_split) else None
            rows = sft_data.load_and_tokenize(src, self.tokenizer, c, split)
            ex.extend(rows)
            self._source_sizes.append(len(rows))
        if not ex:
            raise ValueError("no training examples: set dataset_name / train_datasets / pretokenized_dataset_paths")
        self.train_examples = ex
        return ex

    def load_eval_datasets(self) -> Optional[List[Tuple[str, List[dict]]]]:
        if self.eval_examples is not None:
            return self.eval_examples
        c = self.cfg
        out = []
        names = c.eval_dataset_names or []
        for i, src in enumerate(c.eval_sources()):
            name = names[i] if i < len(names) else os.path.splitext(os.path.basename(src))[0]
            out.append((name, sft_data.load_and_tokenize(src, self.tokenizer, c)))
        for p in (c.eval_pretokenized_dataset_paths or []):
            out.append((os.path.splitext(os.path.basename(p))[0], sft_data.load_pretokenized(p)))
        self.eval_examples = out or None
        return self.eval_examples

    def build_train_sampler(self, examples: List[dict]) -> sft_data.StatefulSampler:
        c = self.cfg
        weights = None
        if c.train_dataset_weights and getattr(self, "_source_sizes", None):
            weights = []
            sizes = self._source_sizes[-len(c.train_dataset_weights):]
            for w, n in zip(c.train_dataset_weights, sizes):
                weights.extend([w / max(n, 1)] * n)
            weights = [0.0] * (len(examples) - len(weights)) + weights if len(weights) < len(examples) else weights
        if c.sampler_class_path:
            import importlib

            mod, _, name = c.sampler_class_path.rpartition(".")
            return getattr(importlib.import_module(mod), name)([len(e["input_ids"]) for e in examples], c.batch_size,
                                                               seed=c.seed, **c.sampler_kwargs)
        return sft_data.StatefulSampler([len(e["input_ids"]) for e in examples], c.batch_size, seed=c.seed, mode=c.sampler,
                                        weights=weights, **c.sampler_kwargs)

    # ------------------------------------------------------------------ one step
    def _local_share(self, batch: TrainingInputBatch) -> TrainingInputBatch:
        """This rank's rows: equal contiguous chunks, or whole bins dealt round-robin when the batch is packed."""
        W, r = self.env.world_size, self.env.rank
        bins = batch.metadata.get("pack_bins")
        if bins:
            starts = [0]
            for b in bins:
                starts.append(starts[-1] + b)
            rows = [i for k in range(r, len(bins), W) for i in range(starts[k], starts[k + 1])]
            if not rows:  # fewer bins than ranks: train on a masked copy so collectives stay matched
                out = batch.slice(0, 1)
                out["loss_mask"] = torch.zeros_like(out["loss_mask"])
                return out
            return batch.select(rows)
        per = batch.batch_size // W
        return batch.slice(r * per, (r + 1) * per)

    def train_step(self, batch: TrainingInputBatch, step: int = 0) -> Dict[str, Any]:
        timings: Dict[str, float] = {}
        total = float(batch["loss_mask"].sum())
        meta = dict(batch.metadata)
        local = self._local_share(batch)
        local.metadata = meta
        local["loss_mask"] = local["loss_mask"].float() / max(total, 1.0)
        t0 = time.perf_counter()
        out = self.policy.forward_backward(local, loss_fn="cross_entropy")
        timings["forward_backward"] = time.perf_counter() - t0
        t0 = time.perf_counter()
        gn = self.policy.optim_step()
        timings["optim_step"] = time.perf_counter() - t0
        # "*loss" metrics are summed over micro-batches and ranks: with the mask pre-divided by the global
        # trained-token count that sum is the token-mean NLL of the whole batch
        return {"loss": float(out.get("policy_loss", float("nan"))), "grad_norm": float(gn) if gn is not None else float("nan"),
                "timings": timings, "trained_tokens": total, "lr": self.policy.get_lr()}

    @torch.no_grad()
    def _run_eval_one(self, examples: List[dict]) -> Tuple[float, int]:
        """Token-mean NLL over one eval set (forward only)."""
        c, W, r = self.cfg, self.env.world_size, self.env.rank
        nll, ntok = 0.0, 0.0
        bs = max(c.batch_size, W)
        for s in range(0, len(examples), bs):
            chunk = examples[s : s + bs]
            while len(chunk) % W:
                chunk = chunk + [dict(chunk[-1], loss_mask=[0] * len(chunk[-1]["loss_mask"]))]
            b = sft_data.collate_sft_batch(chunk, self.tokenizer)
            per = b.batch_size // W
            loc = b.slice(r * per, (r + 1) * per)
            loc.metadata = dict(b.metadata)
            lp = self.policy.forward(loc)["output"]
            m = loc["loss_mask"].float()
            nll += float(-(lp.float().cpu() * m).sum())
            ntok += float(m.sum())
        t = torch.tensor([nll, ntok], dtype=torch.float64)
        if dist.is_initialized() and W > 1:
            t = t.to(self.env.device) if self.env.device.type == "cuda" else t
            dist.all_reduce(t)
        return float(t[0] / max(float(t[1]), 1.0)), int(t[1])

    def run_eval(self) -> Dict[str, float]:
        sets = self.load_eval_datasets()
        if not sets:
            return {}
        out = {}
        for name, ex in sets:
            loss, ntok = self._run_eval_one(ex)
            out[f"eval/{name}/loss"] = loss
            out[f"eval/{name}/tokens"] = float(ntok)
        return out

    # ------------------------------------------------------------------ loop
    def _resolve_num_steps(self, steps_per_epoch: int) -> int:
        c = self.cfg
        n = c.num_steps if c.num_steps is not None else int(math.ceil((c.num_epochs or 1) * steps_per_epoch))
        if c.max_training_steps is not None:
            n = min(n, c.max_training_steps)
        return n

    def _build_dummy_batch(self) -> TrainingInputBatch:
        """Full-context fabricated batch (``dummy_run_full_ctx``): sizes memory and throughput without data."""
        c = self.cfg
        L = c.max_length or 2048
        vocab = self.policy.model.args.vocab_size
        g = torch.Generator().manual_seed(c.seed)
        ex = []
        for _ in range(c.batch_size):
            ids = torch.randint(4, vocab, (L,), generator=g).tolist()
            ex.append({"input_ids": ids, "attention_mask": [1] * L, "loss_mask": [1] * (L - 1), "num_actions": L - 1})
        return sft_data.collate_sft_batch(ex, self.tokenizer)

    def _log(self, metrics: Dict[str, float], step: int) -> None:
        if self.tracker is not None:
            self.tracker.log(metrics, step)

    def train(self) -> Dict[str, float]:
        c = self.cfg
        if self.policy is None:
            self.setup()
        last: Dict[str, float] = {}
        if c.dummy_run_full_ctx:
            batch = self._build_dummy_batch()
            for step in range(1, c.dummy_run_max_steps + 1):
                t0 = time.perf_counter()
                r = self.train_step(batch, step)
                dt = time.perf_counter() - t0
                last = {"train/loss": r["loss"], "train/grad_norm": r["grad_norm"], "timing/step": dt,
                        "train/tokens_per_second": float(batch["attention_mask"].sum()) / dt}
                self._log(last, step)
            return last
        examples = self.load_dataset()
        self.sampler = self.build_train_sampler(examples)
        self.global_step = self.load_checkpoint()
        total = self._resolve_num_steps(len(self.sampler))
        self.total_steps, self.steps_per_epoch, self.epoch = total, len(self.sampler), self.sampler.epoch
        self.callbacks.fire("on_train_start", self)
        if c.eval_before_train and self.global_step == 0:
            ev = self.run_eval()
            if ev:
                self._log(ev, 0)
        done = self.global_step >= total
        while not done:
            self.epoch = self.sampler.epoch
            self.callbacks.fire("on_epoch_start", self)
            for idx in self.sampler:
                t0 = time.perf_counter()
                batch = sft_data.collate_sft_examples([examples[i] for i in idx], self.collator, c.batch_size,
                                                      pad_to_batch_size=not c.use_sequence_packing)
                t_collate = time.perf_counter() - t0
                self.callbacks.fire("on_step_start", self, batch=batch)
                r = self.train_step(batch, self.global_step + 1)
                self.global_step += 1
                dt = time.perf_counter() - t0
                last = {"train/loss": r["loss"], "train/grad_norm": r["grad_norm"], "train/lr": r["lr"],
                        "train/epoch": float(self.sampler.epoch), "train/trained_tokens": r["trained_tokens"],
                        "train/tokens_per_second": float(batch["attention_mask"].sum()) / dt,
                        "timing/step": dt, "timing/collate": t_collate,
                        **{f"timing/{k}": v for k, v in r["timings"].items()}}
                ctl = self.callbacks.fire("on_step_end", self, batch=batch, metrics=last)
                # the flags are read once per step, here; what later events of this step set counts for the next step
                want_save, want_eval_flag, stop = ctl.should_save, ctl.should_evaluate, ctl.should_stop
                ctl.reset()
                if (c.eval_interval > 0 and self.global_step % c.eval_interval == 0) or want_eval_flag:
                    self.callbacks.fire("on_eval_start", self)
                    ev = self.run_eval()
                    last.update(ev)
                    self.callbacks.fire("on_eval_end", self, metrics=ev)
                self.callbacks.fire("on_log", self, logs=last)
                self._log(last, self.global_step)
                if (c.ckpt_interval > 0 and self.global_step % c.ckpt_interval == 0) or want_save:
                    self.save_checkpoint()
                if c.hf_save_interval > 0 and self.global_step % c.hf_save_interval == 0:
                    self.save_hf_model()
                if self.global_step >= total or stop:
                    done = True
                    break
            self.callbacks.fire("on_epoch_end", self)
        if c.ckpt_interval > 0 and c.ckpt_path:
            self.save_checkpoint()
        self.callbacks.fire("on_train_end", self)
        if self.tracker is not None:
            self.tracker.finish()
        return last

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self) -> str:
        c = self.cfg
        if not c.ckpt_path:
            return ""
        d = os.path.join(c.ckpt_path, f"{tutils.GLOBAL_STEP_PREFIX}{self.global_step}")
        os.makedirs(d, exist_ok=True)
        self.policy.save_checkpoint(os.path.join(d, "policy"), tag=str(self.global_step))
        if self.env.is_main:
            torch.save({"global_step": self.global_step, "sampler": self.sampler.state_dict() if self.sampler else None,
                        "config": c.to_dict()}, os.path.join(d, "trainer_state.pt"))
        if dist.is_initialized():
            dist.barrier()
        if self.env.is_main:
            tutils.write_latest(c.ckpt_path, self.global_step)
            tutils.cleanup_old_checkpoints(c.ckpt_path, c.max_ckpts_to_keep, self.global_step)
        self.callbacks.fire("on_save", self, ckpt_path=d)
        return d

    def load_checkpoint(self) -> int:
        c = self.cfg
        if not c.resume_from:
            return 0
        d = c.resume_from
        if d == "latest":
            p = os.path.join(c.ckpt_path, tutils.LATEST_FILE) if c.ckpt_path else ""
            if not p or not os.path.exists(p):
                return 0
            step = int(open(p).read().strip())
            d = os.path.join(c.ckpt_path, f"{tutils.GLOBAL_STEP_PREFIX}{step}")
        state = torch.load(os.path.join(d, "trainer_state.pt"), weights_only=False)
        self.policy.load_checkpoint(os.path.join(d, "policy"))
        if self.sampler is not None and state.get("sampler"):
            self.sampler.load_state_dict(state["sampler"])
        return int(state["global_step"])

    def save_hf_model(self) -> None:
        if self.cfg.export_path:
            self.policy.save_hf_model(os.path.join(self.cfg.export_path, f"{tutils.GLOBAL_STEP_PREFIX}{self.global_step}",
                                                   "policy"), self.tokenizer)

    def shutdown(self) -> None:
        if self.tracker is not None:
            self.tracker.finish()
