"""RL training entry point: ``python -m skyrl_b200.entrypoints.main_base key=value ...``

The experiment object mirrors the reference's overridable hook set (skyrl/train/entrypoints/main_base.py:43-335:
``get_tokenizer / get_train_dataset / get_eval_dataset / get_generator / get_trainer / get_tracker /
get_inference_client / _setup_trainer / run``) so that user subclasses port over by changing the import.  What
differs is the process model: the reference starts a Ray cluster, a placement group and actor groups; here every
GPU already runs this same program (``skyrl_b200.launch`` or ``torch.distributed.run`` starts one process per GPU),
so "placement" is the rank -> GPU identity map and there is nothing to schedule.

For several GPUs::

    python -m skyrl_b200.launch --nproc-per-node 8 -m skyrl_b200.entrypoints.main_base trainer.policy.model.path=...
"""

from __future__ import annotations

import json
import sys
import traceback
from typing import List, Optional

from ..config.config import SkyRLTrainConfig
from ..parallel import dist as pdist
from ..train.dataset import PromptDataset
from ..train.tracking import Tracking
from ..utils.tokenizer import get_tokenizer


class BasePPOExp:
    def __init__(self, cfg: SkyRLTrainConfig):
        self.cfg = cfg
        self.env = pdist.init_distributed()
        self.tokenizer = self.get_tokenizer()
        self.train_dataset = self.get_train_dataset()
        self.eval_dataset = self.get_eval_dataset()

    # ------------------------------------------------------------------ hooks
    @staticmethod
    def get_cfg_as_str(cfg: SkyRLTrainConfig) -> str:
        return json.dumps(cfg.to_dict(), indent=2, default=str)

    def get_tokenizer(self):
        t = self.cfg.trainer
        from ..models.decoder import PRESETS

        vocab = PRESETS[t.policy.model.path].vocab_size if t.policy.model.path in PRESETS else None
        return get_tokenizer(t.policy.model.path, vocab_size=vocab, use_fast=not t.disable_fast_tokenizer)

    def get_train_dataset(self) -> Optional[PromptDataset]:
        d = self.cfg.data
        ds = PromptDataset(d.train_data, self.tokenizer, self.cfg.trainer.max_prompt_length,
                           num_workers=d.dataloader.num_workers or 0)
        if len(ds) < self.cfg.trainer.train_batch_size:
            raise ValueError(f"train dataset has {len(ds)} prompts, fewer than train_batch_size="
                             f"{self.cfg.trainer.train_batch_size}")
        return ds

    def get_eval_dataset(self) -> Optional[PromptDataset]:
        t = self.cfg.trainer
        if t.eval_interval > 0 and self.cfg.data.val_data:
            return PromptDataset(self.cfg.data.val_data, self.tokenizer, t.max_prompt_length)
        return None

    def get_tracker(self) -> Optional[Tracking]:
        t = self.cfg.trainer
        if not self.env.is_main:
            return None
        return Tracking(t.project_name, t.run_name, t.logger, config=self.cfg.to_dict(), log_dir=t.log_path, tags=t.tags)

    def get_inference_client(self):
        """``None`` = colocated engine built by the trainer on this rank's GPU; otherwise a remote client that
        talks to stand-alone servers (``generator.inference_engine.external_server_urls`` / ``external_proxy_url``)."""
        ie = self.cfg.generator.inference_engine
        urls = list(getattr(ie, "external_server_urls", None) or [])
        proxy = getattr(ie, "external_proxy_url", None)
        if not urls and not proxy:
            return None
        from ..inference.remote_client import RemoteInferenceClient

        return RemoteInferenceClient(urls or [proxy], router_url=proxy, tokenizer=self.tokenizer,
                                     model_name=self.cfg.trainer.policy.model.path)

    def get_generator(self, cfg, tokenizer, inference_engine_client):
        """``None`` lets the trainer build the default SkyRL-Gym generator around its engine."""
        if inference_engine_client is None:
            return None
        from ..train.generators.skyrl_gym_generator import SkyRLGymGenerator

        return SkyRLGymGenerator(cfg.generator, cfg.environment.skyrl_gym, inference_engine_client, tokenizer)

    def get_trainer(self, cfg, tracker, tokenizer, train_dataset, eval_dataset, inference_engine_client, generator):
        if cfg.trainer.fully_async.enabled and cfg.trainer.fully_async.simulate_training:
            # rollout-side dry run: generation, staleness control and weight-sync pacing are real, training is a timed stub
            from ..train.fully_async_trainer import FullyAsyncTrainerSim

            cls = FullyAsyncTrainerSim
        elif cfg.trainer.fully_async.enabled:
            from ..train.fully_async_trainer import FullyAsyncPPOTrainer

            cls = FullyAsyncPPOTrainer
        else:
            from ..train.trainer import PPOTrainer

            cls = PPOTrainer
        return cls(cfg, tracker=tracker, tokenizer=tokenizer, train_dataset=train_dataset, eval_dataset=eval_dataset,
                   inference_engine_client=inference_engine_client, generator=generator, env=self.env)

    # ------------------------------------------------------------------ assembly
    def _setup_trainer(self):
        client = self.get_inference_client()
        generator = self.get_generator(self.cfg, self.tokenizer, client)
        tracker = self.get_tracker()
        trainer = self.get_trainer(self.cfg, tracker, self.tokenizer, self.train_dataset, self.eval_dataset, client,
                                   generator)
        trainer.rollout_servers_in_box = bool(getattr(self, "rollout_servers_in_box", False))
        trainer.build_models()
        return trainer

    def run(self):
        trainer = None
        try:
            trainer = self._setup_trainer()
            trainer.train()
        except BaseException as e:  # route the failure to the tracker before the process dies
            tr = getattr(trainer, "tracker", None) if trainer is not None else None
            if tr is not None and not isinstance(e, KeyboardInterrupt):
                try:
                    tr.log_exception(e)
                    tr.finish()
                except Exception:
                    pass
            traceback.print_exc()
            raise
        else:
            tr = getattr(trainer, "tracker", None)
            if tr is not None:
                tr.finish()
        finally:
            pdist.shutdown()
        return trainer


def skyrl_entrypoint(cfg: SkyRLTrainConfig):
    return BasePPOExp(cfg).run()


def _resolve_override_entrypoint(cfg: SkyRLTrainConfig):
    """``trainer.override_entrypoint=pkg.module:Class`` swaps the experiment class without a new launcher."""
    spec = cfg.trainer.override_entrypoint
    if not spec:
        return BasePPOExp
    import importlib

    mod, _, name = spec.partition(":")
    return getattr(importlib.import_module(mod), name or "Exp")


def split_roles(cfg: SkyRLTrainConfig) -> Optional[str]:
    """Disaggregated placement inside one launch (``trainer.placement.colocate_all=false`` with locally run engines):
    the first ``policy_num_gpus_per_node`` ranks train, the remaining ``num_engines`` ranks only serve rollouts.

    The split happens *before* any process group exists: each side becomes its own ``torch.distributed`` world (own
    RANK / WORLD_SIZE / MASTER_PORT; LOCAL_RANK keeps naming the physical GPU), the rollout side runs the serving
    entry point on fixed ports and the training side talks to it like to any stand-alone server -- requests over
    HTTP, weights by peer stores into the servers' exported parameter buffers.  Returns ``"train"``, ``"rollout"`` or
    ``None`` (colocated / single process / external servers).  Reference topology: non-colocated placement of
    skyrl/train/fully_async_trainer.py:392 with weight sync per worker_dispatch.py:693-707."""
    import os

    ie, pl = cfg.generator.inference_engine, cfg.trainer.placement
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if pl.colocate_all or not ie.run_engines_locally or world <= 1 or ie.external_server_urls or ie.external_proxy_url:
        return None
    if "SKYRL_B200_ROLE" in os.environ:  # already split (the environment was rewritten below)
        return os.environ["SKYRL_B200_ROLE"]
    n_train = int(pl.policy_num_gpus_per_node) * int(pl.policy_num_nodes)
    n_roll = int(ie.num_engines) * int(ie.tensor_parallel_size or 1)
    if n_train + n_roll != world:
        raise ValueError(f"disaggregated placement needs policy GPUs ({n_train}) + rollout GPUs ({n_roll}) == world size "
                         f"({world}); set trainer.placement.policy_num_gpus_per_node and generator.inference_engine.num_engines")
    if int(ie.tensor_parallel_size or 1) != 1:
        raise ValueError("rollout-only ranks serve unsharded engines (tensor_parallel_size=1)")
    rank = int(os.environ.get("RANK", "0"))
    port = int(os.environ.get("MASTER_PORT", "29500"))
    base = int(os.environ.get("SKYRL_B200_ROLLOUT_BASE_PORT", str(port + 100)))
    os.environ["SKYRL_B200_ROLLOUT_URLS"] = ",".join(f"http://127.0.0.1:{base + j}" for j in range(n_roll))
    os.environ["SKYRL_B200_ROLLOUT_BASE_PORT"] = str(base)
    if rank < n_train:
        os.environ.update(WORLD_SIZE=str(n_train), RANK=str(rank), SKYRL_B200_ROLE="train")
        return "train"
    os.environ.update(WORLD_SIZE=str(n_roll), RANK=str(rank - n_train), MASTER_PORT=str(port + 1), SKYRL_B200_ROLE="rollout")
    return "rollout"


def _wait_for_servers(urls: List[str], timeout_s: float = 600.0) -> None:
    import time
    import urllib.request

    t0 = time.time()
    pending = list(urls)
    while pending:
        for u in list(pending):
            try:
                with urllib.request.urlopen(u + "/health", timeout=2) as r:
                    if r.status == 200:
                        pending.remove(u)
            except Exception:
                pass
        if pending:
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"rollout servers did not come up: {pending}")
            time.sleep(0.5)


def _shutdown_servers(urls: List[str]) -> None:
    import urllib.request

    for u in urls:
        try:
            urllib.request.urlopen(urllib.request.Request(u + "/skyrl/v1/shutdown", data=b"{}", method="POST"), timeout=5)
        except Exception:
            pass


def main(argv: Optional[List[str]] = None) -> None:
    import os

    cfg = SkyRLTrainConfig.from_cli_overrides(sys.argv[1:] if argv is None else argv)
    role = split_roles(cfg)
    if role == "rollout":
        from .serve import InferenceOnlyEntrypoint

        cfg.trainer.placement.colocate_all = True  # the serving entry point owns its GPU
        InferenceOnlyEntrypoint(cfg, base_port=int(os.environ["SKYRL_B200_ROLLOUT_BASE_PORT"])).run(with_router=False)
        return
    urls: List[str] = []
    if role == "train":
        urls = os.environ["SKYRL_B200_ROLLOUT_URLS"].split(",")
        cfg.generator.inference_engine.external_server_urls = urls
        _wait_for_servers(urls)
    exp = _resolve_override_entrypoint(cfg)(cfg)
    exp.rollout_servers_in_box = role == "train"
    try:
        exp.run()
    finally:
        if role == "train" and int(os.environ.get("RANK", "0")) == 0:
            _shutdown_servers(urls)


if __name__ == "__main__":
    main()
