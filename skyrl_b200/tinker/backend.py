"""Tinker -> trainer adapter: owns the policy (and optional critic) worker and the colocated generation engine of
one base model and executes the engine loop's batched operations on them.

Reference: skyrl/backends/skyrl_train_backend.py:128-1343 (``SkyRLTrainBackend``).  Same behaviours: Tinker datums
arrive already shifted (``model_input`` of length L predicts ``target_tokens`` of length L), so the last target token
is appended to rebuild the full sequence (:647-650); batches are left-padded with right-aligned response tensors;
loss names are normalised (``ppo`` -> ``regular``); the learning rate is set per ``optim_step`` from the request's Adam
parameters; training checkpoints are tar archives; sampler checkpoints either publish the live weights to the
colocated engine (ephemeral) or also persist an HF export.
"""

from __future__ import annotations

import io
import os
import tarfile
import tempfile
import time
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..config.config import SkyRLTrainConfig
from ..parallel.dist import DistEnv, get_env
from ..train.batch import TrainingInputBatch

LOSS_ALIASES = {"ppo": "regular"}
POLICY_LOSSES = ("cross_entropy", "importance_sampling", "ppo", "regular", "gspo", "cispo", "dppo", "dual_clip", "sapo")


def tensor_data(values: List[float], dtype: str = "float32") -> Dict[str, Any]:
    return {"data": list(values), "dtype": dtype, "shape": [len(values)]}


def flatten_model_input(model_input: Dict[str, Any]) -> List[int]:
    """Token ids of a ``ModelInput`` (text chunks only; image chunks need a multimodal renderer)."""
    ids: List[int] = []
    for ch in model_input.get("chunks", []):
        if "tokens" not in ch:
            raise ValueError("image chunks are not supported by this text-only backend")
        ids.extend(int(t) for t in ch["tokens"])
    return ids


def datums_to_batch(datums: List[Dict[str, Any]], pad_token_id: int, role: str = "policy") -> TrainingInputBatch:
    seqs, weights, lps, advs, vals, rets = [], [], [], [], [], []
    for d in datums:
        ids = flatten_model_input(d["model_input"])
        li = d.get("loss_fn_inputs", {})
        tg = [int(x) for x in (li.get("target_tokens") or {}).get("data", [])]
        w = [float(x) for x in (li.get("weights") or {}).get("data", [])] or [1.0] * len(tg)
        if len(tg) != len(ids) or len(w) != len(tg):
            raise ValueError(f"datum has {len(ids)} input tokens, {len(tg)} targets and {len(w)} weights; they must match")
        seqs.append(ids + ([tg[-1]] if tg else []))
        weights.append(w)
        lps.append([float(x) for x in (li.get("logprobs") or {}).get("data", [])])
        advs.append([float(x) for x in (li.get("advantages") or {}).get("data", [])])
        vals.append([float(x) for x in (li.get("values") or {}).get("data", [])])
        rets.append([float(x) for x in (li.get("returns") or {}).get("data", [])])
    S = max(len(s) for s in seqs)
    R = max(len(w) for w in weights)
    n = len(seqs)
    sequences = torch.full((n, S), pad_token_id, dtype=torch.long)
    att = torch.zeros((n, S), dtype=torch.long)
    lmask, rmask = torch.zeros((n, R)), torch.zeros((n, R), dtype=torch.long)

    def right(rows, need_all: bool) -> Optional[torch.Tensor]:
        if not any(rows):
            return None
        out = torch.zeros((n, R))
        for i, r in enumerate(rows):
            if r:
                if len(r) != len(weights[i]):
                    raise ValueError("per-token loss inputs must have one value per target token")
                out[i, R - len(r):] = torch.tensor(r)
            elif need_all:
                raise ValueError("either every datum or none carries this loss input")
        return out

    for i, (s, w) in enumerate(zip(seqs, weights)):
        sequences[i, S - len(s):] = torch.tensor(s)
        att[i, S - len(s):] = 1
        lmask[i, R - len(w):] = torch.tensor(w)
        rmask[i, R - len(w):] = 1
    d: Dict[str, Any] = {"sequences": sequences, "attention_mask": att, "loss_mask": lmask, "response_mask": rmask}
    lp_t, adv_t = right(lps, False), right(advs, False)
    if lp_t is not None:
        d["action_log_probs"] = lp_t
        d["rollout_logprobs"] = lp_t.clone()
    if adv_t is not None:
        d["advantages"] = adv_t
    if role == "critic":
        v_t, r_t = right(vals, True), right(rets, True)
        if (v_t is None) != (r_t is None):
            raise ValueError("critic batches must provide both values and returns, or neither")
        if v_t is not None:
            d["values"], d["returns"] = v_t, r_t
    b = TrainingInputBatch(d)
    b.metadata = {"response_length": R}
    return b


class ModelSlot:
    """One Tinker ``model_id``: a worker plus bookkeeping.  ``store`` is set for LoRA models: they are tenants of an
    ``AdapterStore`` on a worker that several model ids share (one resident base model, one adapter + optimizer state
    per id, swapped in before every verb)."""

    def __init__(self, model_id: str, worker, role: str, lora_config: Optional[dict], store=None):
        self.model_id, self.worker, self.role, self.lora_config, self.store = model_id, worker, role, lora_config, store
        self.step = 0
        self.sampler_version = 0


class SkyRLTrainBackend:
    def __init__(self, base_model: str, overrides: Optional[Dict[str, Any]] = None, env: Optional[DistEnv] = None,
                 tokenizer=None, checkpoints_base: Optional[str] = None):
        args = [f"trainer.policy.model.path={base_model}", "trainer.logger=console", "trainer.resume_mode=none"]
        for k, v in (overrides or {}).items():
            args.append(f"{k}={v}")
        self.cfg = SkyRLTrainConfig.from_cli_overrides(args)
        self.base_model = base_model
        self.env = env or get_env()
        self.tokenizer = tokenizer
        self.models: Dict[str, ModelSlot] = {}
        self._lora_hosts: Dict[tuple, Any] = {}  # (rank, alpha) -> AdapterStore whose worker holds the shared base model
        self.engine = None
        self._engine_owner = None  # the worker whose ``engine_model()`` the engine runs
        self.client = None
        self.sampler_version = 0
        self.checkpoints_base = checkpoints_base or os.path.join(tempfile.gettempdir(), "skyrl_b200_tinker")
        os.makedirs(self.checkpoints_base, exist_ok=True)

    # ------------------------------------------------------------------ lifecycle
    def _pad_id(self) -> int:
        t = self.tokenizer
        return t.pad_token_id if t is not None and getattr(t, "pad_token_id", None) is not None else 0

    def has_model(self, model_id: str) -> bool:
        return model_id in self.models

    def create_model(self, model_id: str, lora_config: Optional[dict] = None, model_role: str = "policy") -> None:
        from ..workers.worker import CriticWorker, PolicyWorker

        if model_id in self.models:
            raise ValueError(f"model {model_id} already exists")
        t = self.cfg.trainer
        seed = int((lora_config or {}).get("seed") or t.seed)
        rank = int((lora_config or {}).get("rank") or 0)
        if model_role == "critic":
            w = CriticWorker(t, model_path=t.critic.model.path or self.base_model, env=self.env, seed=seed)
            self.models[model_id] = ModelSlot(model_id, w, model_role, lora_config)
            return
        if rank > 0:
            # LoRA models of one shape share a worker: the frozen base is resident once, each model id owns an adapter
            # buffer, its fp32 master copy, Adam moments and pending gradients (reference: the Megatron backend's
            # AdapterStore and the JAX backend's adapter-indexed LoRA layers)
            from ..workers.adapter_store import AdapterStore

            alpha = float((lora_config or {}).get("alpha") or t.policy.model.lora.alpha)
            key = (rank, alpha)
            store = self._lora_hosts.get(key)
            if store is None:
                import copy

                tc = copy.deepcopy(t)
                tc.policy.model.lora.rank, tc.policy.model.lora.alpha = rank, alpha
                w = PolicyWorker(tc, model_path=self.base_model, env=self.env, seed=int(t.seed))
                store = AdapterStore(w, max_slots=max(1, int(t.policy.model.lora.max_loras or 1), self.max_lora_models))
                self._lora_hosts[key] = store
            store.create(model_id, seed=seed)
            self.models[model_id] = ModelSlot(model_id, store.worker, model_role, lora_config, store=store)
            return
        w = PolicyWorker(t, model_path=self.base_model, env=self.env, seed=seed)
        self.models[model_id] = ModelSlot(model_id, w, model_role, lora_config)

    max_lora_models = 16  # tenants per shared base; their state lives in pinned host memory while inactive

    def _activate(self, slot: ModelSlot) -> None:
        """Bring the model id's adapter (with optimizer state and pending gradients) into its worker."""
        if slot.store is not None:
            slot.store.swap_to(slot.model_id)

    def delete_model(self, model_id: str) -> None:
        slot = self.models.pop(model_id, None)
        if slot is None:
            return
        last_user = True
        if slot.store is not None:
            slot.store.delete(model_id)
            last_user = not slot.store.slots
            if last_user:
                self._lora_hosts = {k: v for k, v in self._lora_hosts.items() if v is not slot.store}
        if last_user and self.engine is not None and self._engine_owner is slot.worker:
            self.engine, self.client, self._engine_owner = None, None, None
        del slot
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    @staticmethod
    def normalize_loss_fn_config(loss_fn: str, cfg: Optional[dict]) -> Optional[dict]:
        """Tinker's per-request knobs -> fields of the algorithm config (reference: skyrl_train_backend.py:840-872).
        Ratio thresholds are centred on one (``clip_low_threshold=0.9`` means ``eps_clip_low=0.1``); DPPO's deltas and
        CISPO's clips live in their nested sections; anything else (``value_clip``) keeps its name."""
        if not cfg:
            return None
        out = dict(cfg)
        lo, hi = out.pop("clip_low_threshold", None), out.pop("clip_high_threshold", None)
        if loss_fn == "cispo":
            nested = {}
            if lo is not None:
                nested["cispo_eps_clip_low"] = 1.0 - float(lo)
            if hi is not None:
                nested["cispo_eps_clip_high"] = float(hi) - 1.0
            if nested:
                out["cispo"] = nested
        else:
            if lo is not None:
                out["eps_clip_low"] = 1.0 - float(lo)
            if hi is not None:
                out["eps_clip_high"] = float(hi) - 1.0
        if loss_fn == "dppo":
            nested = {k: float(out.pop(k)) for k in ("delta_low", "delta_high") if k in out}
            if nested:
                out["dppo"] = nested
        return out or None

    # ------------------------------------------------------------------ training verbs
    def forward_backward(self, model_id: str, datums: List[dict], loss_fn: str, loss_fn_config: Optional[dict] = None,
                         forward_only: bool = False) -> Dict[str, Any]:
        slot = self.models[model_id]
        self._activate(slot)
        batch = datums_to_batch(datums, self._pad_id(), slot.role)
        name = LOSS_ALIASES.get(loss_fn, loss_fn)
        loss_fn_config = self.normalize_loss_fn_config(loss_fn, loss_fn_config)
        if slot.role == "critic" and loss_fn not in ("ppo", "ppo_critic"):
            raise ValueError(f"critic models take loss_fn 'ppo' or 'ppo_critic', got '{loss_fn}'")
        if slot.role != "critic" and loss_fn == "ppo_critic":
            raise ValueError("loss_fn 'ppo_critic' is only valid for critic models")
        if slot.role == "critic" or name == "ppo_critic":
            if forward_only:
                vals = slot.worker.forward(batch)["output"]
                outs = self._per_row(vals, batch, "values")
                return {"loss_fn_output_type": "values", "loss_fn_outputs": outs, "metrics": {}}
            algo = slot.worker.cfg.algorithm
            keep = algo.value_clip
            if loss_fn_config and "value_clip" in loss_fn_config:
                algo.value_clip = float(loss_fn_config["value_clip"])
            try:
                st = slot.worker.forward_backward(batch)
            finally:
                algo.value_clip = keep
            return {"loss_fn_output_type": "scalar", "loss_fn_outputs": [], "metrics": self._metrics(st)}
        if forward_only:
            lp = slot.worker.forward(batch)["output"]
            outs = self._per_row(lp, batch, "logprobs", with_loss=(name == "cross_entropy"))
            return {"loss_fn_output_type": "logprobs", "loss_fn_outputs": outs, "metrics": {}}
        st = slot.worker.forward_backward(batch, loss_fn=name, loss_fn_config=loss_fn_config, return_per_token_outputs=True)
        outs = []
        for o in st.pop("loss_fn_outputs", []):
            row = {"logprobs": tensor_data(o["logprobs"])}
            if "elementwise_loss" in o:
                row["elementwise_loss"] = tensor_data(o["elementwise_loss"])
            outs.append(row)
        return {"loss_fn_output_type": "logprobs", "loss_fn_outputs": outs, "metrics": self._metrics(st)}

    @staticmethod
    def _per_row(t: torch.Tensor, batch: TrainingInputBatch, key: str, with_loss: bool = False) -> List[dict]:
        rm, lm = batch["response_mask"], batch["loss_mask"]
        R = rm.shape[1]
        outs = []
        t = t.float().cpu()
        for i in range(rm.shape[0]):
            n = int(rm[i].sum())
            row = t[i, R - n:].tolist() if n else []
            o = {key: tensor_data(row)}
            if with_loss:
                o["elementwise_loss"] = tensor_data([-a * b for a, b in zip(row, lm[i, R - n:].tolist())])
            outs.append(o)
        return outs

    @staticmethod
    def _metrics(st: Dict[str, Any]) -> Dict[str, float]:
        out = {}
        for k, v in st.items():
            if isinstance(v, (int, float)):
                out[k.replace("/", ":")] = float(v)
        if "final_loss" in out:
            out["loss:sum"] = out["final_loss"]
        return out

    def optim_step(self, model_id: str, adam_params: Optional[dict] = None) -> Dict[str, Any]:
        slot = self.models[model_id]
        self._activate(slot)
        ap = adam_params or {}
        opt = slot.worker.optimizer
        if "learning_rate" in ap:
            slot.worker.set_lr(float(ap["learning_rate"]))
        if "beta1" in ap or "beta2" in ap:
            opt.betas = (float(ap.get("beta1", opt.betas[0])), float(ap.get("beta2", opt.betas[1])))
        if "eps" in ap:
            opt.eps = float(ap["eps"])
        if "weight_decay" in ap:
            opt.weight_decay = float(ap["weight_decay"])
        applied_lr = slot.worker.get_lr()  # the scheduler may move the value for the following step
        gn = slot.worker.optim_step()
        slot.step += 1
        return {"metrics": {"grad_norm": float(gn) if gn is not None else 0.0, "learning_rate": applied_lr,
                            "step": float(slot.step)}}

    # ------------------------------------------------------------------ sampling
    def _ensure_engine(self, model_id: Optional[str]):
        """The generation engine reads the policy's parameters in place, so publishing weights is a version bump."""
        from ..engine.llm_engine import EngineConfig, LLMEngine

        slot = self.models.get(model_id) if model_id else None
        if slot is None:
            slot = next((s for s in self.models.values() if s.role == "policy"), None)
        if slot is None:
            raise ValueError("no policy model is loaded to sample from")
        self._activate(slot)
        if self.engine is None or self._engine_owner is not slot.worker:
            ie = self.cfg.generator.inference_engine
            g = self.cfg.generator
            max_len = (g.max_input_length or self.cfg.trainer.max_prompt_length) + g.sampling_params.max_generate_length
            eos = [self.tokenizer.eos_token_id] if self.tokenizer is not None and self.tokenizer.eos_token_id is not None else []
            ecfg = EngineConfig(block_size=self.cfg.trainer.b200.kv_block_size, max_num_seqs=ie.max_num_seqs,
                                gpu_memory_utilization=ie.gpu_memory_utilization, max_model_len=max_len,
                                max_num_batched_tokens=max(ie.max_num_batched_tokens, max_len),
                                enforce_eager=ie.enforce_eager, seed=self.cfg.trainer.seed)
            for k, v in (ie.engine_init_kwargs or {}).items():
                if hasattr(ecfg, k):
                    setattr(ecfg, k, v)
            # full-parameter models are read in place; LoRA models run a merged copy that follows the active adapter
            self.engine = LLMEngine(slot.worker.engine_model(), ecfg, eos_token_ids=eos)
            self._engine_owner = slot.worker
        return self.engine

    def sample(self, prompts: List[List[int]], sampling_params: List[dict], num_samples: List[int],
               model_id: Optional[str] = None, prompt_logprobs: bool = False) -> List[Dict[str, Any]]:
        """One result per request: ``{"sequences": [{tokens, logprobs, stop_reason}], "prompt_logprobs": ...}``."""
        from ..engine.llm_engine import SamplingParams

        eng = self._ensure_engine(model_id)
        flat_prompts, flat_params, owner = [], [], []
        for i, (p, sp, n) in enumerate(zip(prompts, sampling_params, num_samples)):
            stop = sp.get("stop")
            stop_ids = [int(s) for s in stop] if stop and all(isinstance(s, int) for s in stop) else None
            stop_str = [s for s in stop if isinstance(s, str)] if stop and stop_ids is None else None
            params = SamplingParams(max_tokens=int(sp.get("max_tokens") or 256), temperature=float(sp.get("temperature", 1.0)),
                                    top_p=float(sp.get("top_p", 1.0)), top_k=int(sp.get("top_k", -1)), stop=stop_str,
                                    stop_token_ids=stop_ids, prompt_logprobs=bool(prompt_logprobs))
            for _ in range(max(1, int(n))):
                flat_prompts.append(p)
                flat_params.append(params)
                owner.append(i)
        # cached prefixes are only shared between requests that see the same weights
        outs = eng.generate(flat_prompts, flat_params, cache_salt=f"{model_id or ''}-v{self.sampler_version}")
        results: List[Dict[str, Any]] = [{"sequences": [], "prompt_logprobs": None, "type": "sample"} for _ in prompts]
        for o, i in zip(outs, owner):
            results[i]["sequences"].append({"tokens": list(o.token_ids), "logprobs": [float(x) for x in o.logprobs],
                                            "stop_reason": "stop" if o.finish_reason == "stop" else "length"})
            if prompt_logprobs and getattr(o, "prompt_logprobs", None) is not None:
                results[i]["prompt_logprobs"] = [None] + [float(x) for x in o.prompt_logprobs]
        return results

    # ------------------------------------------------------------------ checkpoints
    def _ckpt_path(self, model_id: str, checkpoint_id: str, kind: str) -> str:
        d = os.path.join(self.checkpoints_base, model_id, kind)
        os.makedirs(d, exist_ok=True)
        return os.path.join(d, f"{checkpoint_id}.tar")

    def save_checkpoint(self, model_id: str, checkpoint_id: str) -> str:
        """Training state (parameters, optimizer shards, scheduler) as one tar archive."""
        slot = self.models[model_id]
        self._activate(slot)
        out = self._ckpt_path(model_id, checkpoint_id, "weights")
        with tempfile.TemporaryDirectory() as tmp:
            slot.worker.save_checkpoint(tmp, tag=checkpoint_id)
            if self.env.is_main:
                part = out + ".part"
                with tarfile.open(part, "w") as tar:
                    tar.add(tmp, arcname=".")
                os.replace(part, out)
        return out

    def load_checkpoint(self, model_id: str, path: str, optimizer: bool = True) -> None:
        slot = self.models[model_id]
        self._activate(slot)
        with tempfile.TemporaryDirectory() as tmp:
            with tarfile.open(path, "r") as tar:
                tar.extractall(tmp, filter="data")
            slot.worker.load_checkpoint(tmp, load_optimizer_states=optimizer, load_lr_scheduler_states=optimizer)
        self.sampler_version += 1
        slot.worker.refresh_engine_model()
        if self.engine is not None and self._engine_owner is slot.worker:
            self.engine.reset_prefix_cache()
            self.engine.weight_version = self.sampler_version

    def save_sampler_checkpoint(self, model_id: str, checkpoint_id: Optional[str], persist: bool = True) -> Optional[str]:
        """Make the current weights the ones ``sample`` uses.  The colocated engine shares the parameter buffer, so
        this only advances the weight version (which salts the prefix cache); with ``persist`` an HF export is also
        archived so the checkpoint can be downloaded or loaded elsewhere."""
        slot = self.models[model_id]
        self.sampler_version += 1
        eng = self._ensure_engine(model_id)
        slot.worker.refresh_engine_model()  # LoRA: merge the trained adapter into the engine's copy
        eng.reset_prefix_cache()
        eng.weight_version = self.sampler_version
        if not persist or not checkpoint_id:
            return None
        out = self._ckpt_path(model_id, checkpoint_id, "sampler_weights")
        with tempfile.TemporaryDirectory() as tmp:
            slot.worker.save_hf_model(tmp, self.tokenizer)
            if self.env.is_main:
                part = out + ".part"
                with tarfile.open(part, "w") as tar:
                    tar.add(tmp, arcname=".")
                os.replace(part, out)
        return out
