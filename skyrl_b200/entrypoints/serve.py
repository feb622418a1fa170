"""Stand-alone rollout serving: one engine + HTTP server per GPU and, on rank 0, a session-affine router in front
(reference: skyrl/train/entrypoints/serve.py:33-124).  Trainers on another machine point
``generator.inference_engine.external_proxy_url`` / ``external_server_urls`` at the printed addresses.

    python -m skyrl_b200.launch --nproc-per-node 8 -m skyrl_b200.entrypoints.serve trainer.policy.model.path=... \\
        generator.inference_engine.served_model_name=policy

Every rank prints one JSON line ``{"rank", "server_url"}``; rank 0 also prints ``{"router_url", "server_urls"}``.
"""

from __future__ import annotations

import json
import signal
import sys
import threading
from typing import List, Optional

import torch
import torch.distributed as dist

from ..config.config import ConfigError, SkyRLTrainConfig
from ..parallel import dist as pdist
from .main_base import BasePPOExp


def _validate_serve_cfg(cfg: SkyRLTrainConfig) -> None:
    ie = cfg.generator.inference_engine
    if ie.external_proxy_url or ie.external_server_urls:
        raise ConfigError("serve starts its own servers: unset generator.inference_engine.external_proxy_url / "
                          "external_server_urls")
    if not cfg.trainer.policy.model.path:
        raise ConfigError("serve needs trainer.policy.model.path (the model to serve)")


class InferenceOnlyEntrypoint(BasePPOExp):
    def __init__(self, cfg: SkyRLTrainConfig, base_port: int = 0, host: str = "127.0.0.1"):
        _validate_serve_cfg(cfg)
        self.host, self.base_port = host, base_port
        self._servers, self._router = [], None
        self._stop = threading.Event()
        super().__init__(cfg)

    def get_train_dataset(self):
        return None

    def get_eval_dataset(self):
        return None

    def _teardown(self) -> None:
        for s in self._servers:
            s.stop()
        if self._router is not None:
            self._router.stop()
        self._servers, self._router = [], None

    def start(self, with_router: bool = True) -> dict:
        """Bring the servers up and return the address record (does not block)."""
        from ..engine.llm_engine import LLMEngine
        from ..inference.local_client import LocalInferenceClient
        from ..inference.router import SessionRouter, build_router_app
        from ..inference.server import ServerThread, build_app
        from ..models.decoder import build_model
        from ..train.trainer import PPOTrainer

        t = self.cfg.trainer
        dtype = torch.bfloat16 if self.env.device.type == "cuda" else torch.float32
        flat, handle = None, None
        if self.env.device.type == "cuda":
            # the parameter buffer lives in its own allocation so that trainers on other GPUs of the machine can map it
            # and push new weights into it (CUDA IPC; see weight_sync/remote.py, transport "peer")
            from ..models.decoder import flat_numel_for, resolve_model_args
            from ..parallel.peer import ipc_alloc_tensor

            flat, handle, _ = ipc_alloc_tensor(flat_numel_for(resolve_model_args(t.policy.model.path)), dtype, self.env.device)
        model = build_model(t.policy.model.path, device=self.env.device, dtype=dtype, seed=t.seed, flat_buffer=flat)
        shell = PPOTrainer.__new__(PPOTrainer)  # reuse the trainer's engine sizing rules without building workers
        shell.cfg, shell.env, shell.tokenizer = self.cfg, self.env, self.tokenizer
        engine: LLMEngine = shell._build_engine(model)
        client = LocalInferenceClient([engine], self.tokenizer)
        name = getattr(self.cfg.generator.inference_engine, "served_model_name", None) or t.policy.model.path
        port = self.base_port + self.env.rank if self.base_port else 0
        from ..weight_sync.remote import make_weight_loader

        dcfg = self.cfg.generator.inference_engine.delta_weight_sync
        loader = make_weight_loader(model, engine, sync_dir=getattr(dcfg, "sync_dir", "") or None,
                                    local_dir=getattr(dcfg, "local_checkpoint_dir", None), ipc_handle=handle)
        app = build_app(client, model_name=name, weight_loader=loader)

        @app.post("/skyrl/v1/shutdown")
        async def shutdown():  # lets the trainer of a combined train + rollout launch end the rollout ranks
            self._stop.set()
            return {"status": "stopping"}

        srv = ServerThread(app, host=self.host, port=port).start()
        self._servers.append(srv)
        rec = {"rank": self.env.rank, "server_url": srv.url}
        urls = [srv.url]
        if dist.is_initialized() and self.env.world_size > 1:
            gathered: List[Optional[str]] = [None] * self.env.world_size
            dist.all_gather_object(gathered, srv.url)
            urls = [u for u in gathered if u]
        if self.env.is_main and with_router:
            # generator.inference_engine.router_init_kwargs: policy (consistent_hash | sticky_least_loaded |
            # round_robin) and vnodes reach the router; other names belong to the reference's router and are ignored
            rk = {k: v for k, v in (self.cfg.generator.inference_engine.router_init_kwargs or {}).items()
                  if k in ("policy", "vnodes")}
            self._router = ServerThread(build_router_app(SessionRouter(urls, **rk)), host=self.host,
                                        port=(self.base_port + self.env.world_size) if self.base_port else 0).start()
            rec.update({"router_url": self._router.url, "server_urls": urls})
        print(json.dumps(rec), flush=True)
        return rec

    def run(self, with_router: bool = True) -> None:
        self.start(with_router)
        for sig in (signal.SIGINT, signal.SIGTERM):
            try:
                signal.signal(sig, lambda *_: self._stop.set())
            except ValueError:  # not the main thread
                pass
        try:
            self._stop.wait()
        finally:
            self._teardown()
            pdist.shutdown()


def skyrl_entrypoint(cfg: SkyRLTrainConfig):
    InferenceOnlyEntrypoint(cfg).run()


def main(argv: Optional[List[str]] = None) -> None:
    cfg = SkyRLTrainConfig.from_cli_overrides(sys.argv[1:] if argv is None else argv)
    skyrl_entrypoint(cfg)


if __name__ == "__main__":
    main()
