"""``RemoteBackendTrainer``: the PPO / GRPO loop of ``skyrl_b200.train.trainer.PPOTrainer`` with every model operation
(old log-probs, loss + backward, optimizer step, sampling) executed by a training service.

Division of labour (the one of the reference's ``ArcticPPOTrainer``, integrations/arctic_rl/trainer.py:65-157): the
service owns the weights, the surrogate loss and the optimizer; this process owns prompts, environments and rewards,
the advantage estimate, mini-batching and logging.  Nothing here touches a GPU.
"""

from __future__ import annotations

import asyncio
from typing import Any, Dict, List, Optional

import torch

from ...train.generators.skyrl_gym_generator import SkyRLGymGenerator
from ...inference.base import InferenceEngineInput, InferenceEngineInterface, InferenceEngineOutput
from ...train.batch import TrainingInputBatch
from ...train.trainer import PPOTrainer
from .client import TrainingServiceClient

LOSS_NAMES = {"regular": "ppo"}  # this package's name -> the service's name, where they differ


def _tensor(data: List[float], dtype: str) -> Dict[str, Any]:
    return {"data": data, "dtype": dtype, "shape": [len(data)]}


def batch_to_datums(batch: TrainingInputBatch, with_loss_inputs: bool = True) -> List[dict]:
    """One datum per row: the row's real tokens (padding removed), next-token targets, and per-target loss inputs that
    are zero over the prompt (weights = loss mask, old log-probs, advantages)."""
    seqs, att = batch["sequences"], batch["attention_mask"]
    rmask = batch["response_mask"]
    out = []
    for i in range(seqs.shape[0]):
        ids = seqs[i][att[i].bool()].tolist()
        n_resp = int(rmask[i].sum())
        L = len(ids) - 1
        lead = [0.0] * (L - n_resp)
        li = {"target_tokens": _tensor(ids[1:], "int64"),
              "weights": _tensor(lead + batch["loss_mask"][i, :n_resp].float().tolist(), "float32")}
        if with_loss_inputs:
            for key, name in (("action_log_probs", "logprobs"), ("advantages", "advantages")):
                v = batch.get(key)
                if v is not None:
                    li[name] = _tensor(lead + v[i, :n_resp].float().tolist(), "float32")
        out.append({"model_input": {"chunks": [{"type": "encoded_text", "tokens": ids[:-1]}]}, "loss_fn_inputs": li})
    return out


def _response_rows(outputs: List[dict], key: str, batch: TrainingInputBatch) -> torch.Tensor:
    """Per-target service outputs -> ``[B, R]`` aligned with the batch's response columns."""
    R = batch["response_mask"].shape[1]
    res = torch.zeros((len(outputs), R))
    for i, o in enumerate(outputs):
        n_resp = int(batch["response_mask"][i].sum())
        if n_resp:
            res[i, :n_resp] = torch.tensor(o[key]["data"][-n_resp:])
    return res


class RemotePolicyWorker:
    """The worker interface the trainer drives (``forward`` / ``forward_backward`` / ``optim_step`` / checkpoints),
    answered by the service."""

    tp_size = 1

    def __init__(self, cfg, client: TrainingServiceClient):
        self.cfg, self.client = cfg, client
        self._pending: List[Dict[str, Any]] = []
        self._saved = 0

    def forward(self, batch: TrainingInputBatch, train_packing: bool = False) -> Dict[str, torch.Tensor]:
        out = self.client.forward(batch_to_datums(batch, with_loss_inputs=False), "cross_entropy")
        return {"output": _response_rows(out["loss_fn_outputs"], "logprobs", batch)}

    def forward_backward(self, batch: TrainingInputBatch, **_) -> Dict[str, float]:
        a = self.cfg.trainer.algorithm
        loss = LOSS_NAMES.get(a.policy_loss_type, a.policy_loss_type)
        # the service takes Tinker's names: ratio thresholds centred on one for the clipped objectives, deltas for DPPO
        if loss in ("ppo", "gspo"):
            cfg = {"clip_low_threshold": 1.0 - a.eps_clip_low, "clip_high_threshold": 1.0 + a.eps_clip_high}
        elif loss == "cispo":
            cfg = {"clip_low_threshold": 1.0 - a.cispo.cispo_eps_clip_low, "clip_high_threshold": 1.0 + a.cispo.cispo_eps_clip_high}
        elif loss == "dppo":
            cfg = {"delta_low": a.dppo.delta_low, "delta_high": a.dppo.delta_high}
        else:
            cfg = None
        # queued, not awaited: the service runs a model's requests in order, so the optimizer step can be sent behind it
        self._pending.append(self.client.forward_backward_async(batch_to_datums(batch), loss, cfg))
        return {}

    def optim_step(self) -> Optional[float]:
        step = self.client.optim_step_async(self.cfg.trainer.policy.optimizer_config.lr)
        status: Dict[str, float] = {}
        for fut in self._pending:
            for k, v in (self.client.wait(fut).get("metrics") or {}).items():
                if isinstance(v, (int, float)):
                    status[k] = float(v)
        self._pending = []
        m = self.client.wait(step).get("metrics") or {}
        self.last_status = {**status, **{k: float(v) for k, v in m.items() if isinstance(v, (int, float))}}
        return self.last_status.get("grad_norm")

    # checkpoints live on the service; the trainer's directory only records their names
    def save_checkpoint(self, path: str, tag: str = "") -> None:
        import os

        self._saved += 1
        name = self.client.save_state(f"step-{tag or self._saved}")
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "remote_checkpoint.txt"), "w") as f:
            f.write(name)

    def load_checkpoint(self, path: str) -> None:
        import os

        with open(os.path.join(path, "remote_checkpoint.txt")) as f:
            self.client.load_state(f.read().strip())

    def save_hf_model(self, path: str, tokenizer=None) -> None:
        raise NotImplementedError("the service owns the weights: download its checkpoint archive instead")

    def start_profile(self) -> None: ...
    def profile_step(self) -> None: ...
    def stop_profile(self) -> str:
        return ""


class RemoteSamplerClient(InferenceEngineInterface):
    """Token-in / token-out generation through the service's sampler (one request per prompt, all in flight at once)."""

    def __init__(self, client: TrainingServiceClient, tokenizer=None):
        self.client, self.tokenizer = client, tokenizer

    async def generate(self, input_batch: InferenceEngineInput) -> InferenceEngineOutput:
        sp = dict(input_batch.get("sampling_params") or {})
        params = {"max_tokens": int(sp.get("max_generate_length", sp.get("max_tokens", 16))),
                  "temperature": float(sp.get("temperature", 1.0))}
        for k in ("top_p", "top_k", "stop", "seed"):
            if sp.get(k) is not None:
                params[k] = sp[k]
        loop = asyncio.get_running_loop()
        futs = [self.client.sample_async(p, 1, params) for p in input_batch["prompt_token_ids"]]
        res = await loop.run_in_executor(None, lambda: [self.client.wait(f) for f in futs])
        ids = [r["sequences"][0]["tokens"] for r in res]
        text = [self.tokenizer.decode(t) if self.tokenizer is not None else "" for t in ids]
        return {"responses": text, "response_ids": ids, "stop_reasons": [r["sequences"][0]["stop_reason"] for r in res],
                "response_logprobs": [r["sequences"][0].get("logprobs") for r in res]}

    async def pause(self, mode: str = "keep", clear_cache: bool = False) -> None: ...
    async def resume(self) -> None: ...
    async def sleep(self, level: int = 2, tags=None) -> None: ...
    async def wake_up(self, tags=None) -> None: ...
    async def reset_prefix_cache(self, reset_running_requests: bool = False) -> None: ...


class RemoteBackendTrainer(PPOTrainer):
    """``PPOTrainer`` without local models.  Critic, reference model and KL terms need local workers and are rejected."""

    def __init__(self, cfg, client: TrainingServiceClient, **kw):
        a = cfg.trainer.algorithm
        if a.use_kl_loss or a.use_kl_in_reward or a.advantage_estimator == "gae":
            raise ValueError("the remote backend trains a policy only: no reference model, KL term or critic")
        super().__init__(cfg, **kw)
        self.client = client

    def build_models(self, policy_model=None, peer_ctx=None) -> None:
        t = self.cfg.trainer
        if self.client.model_id is None:
            self.client.connect(t.policy.model.path, t.policy.model.lora.rank)
        self.policy = RemotePolicyWorker(self.cfg, self.client)
        self.inference_engine_client = RemoteSamplerClient(self.client, self.tokenizer)
        if self.generator is None:
            self.generator = SkyRLGymGenerator(self.cfg.generator, self.cfg.environment.skyrl_gym,
                                               self.inference_engine_client, self.tokenizer)

    def _old_logprobs_from_train_forward(self) -> bool:
        return False  # the service's loss takes the old log-probs as an input

    def sync_weights(self) -> None:
        """New weights reach the sampler when the service snapshots them under a fresh sampling session."""
        self.client.save_weights_for_sampler()

    async def sync_weights_async(self) -> None:
        await asyncio.get_running_loop().run_in_executor(None, self.sync_weights)

    def train_critic_and_policy(self, batch: TrainingInputBatch) -> Dict[str, float]:
        m = super().train_critic_and_policy(batch)
        for k, v in getattr(self.policy, "last_status", {}).items():
            if f"policy/{k}" not in self.all_metrics:  # what this process measured itself wins
                m.setdefault(f"policy/{k}", v)
        return m
