"""Experiment tracking multiplexer: console, tensorboard, wandb, mlflow, swanlab -- whichever of the
optional packages is importable (reference: skyrl/train/utils/tracking.py:33-292)."""

from __future__ import annotations

import json
import os
import time
import traceback
from typing import Any, Dict, List, Optional, Union


class _Console:
    def log(self, data: Dict[str, Any], step: int) -> None:
        keys = sorted(data)
        body = " | ".join(f"{k}={data[k]:.5g}" if isinstance(data[k], (int, float)) else f"{k}={data[k]}" for k in keys)
        print(f"[step {step}] {body}", flush=True)

    def finish(self) -> None:
        return None


class _Jsonl:
    def __init__(self, path: str):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.f = open(path, "a")

    def log(self, data, step):
        self.f.write(json.dumps({"step": step, "time": time.time(), **{k: v for k, v in data.items()
                                                                        if isinstance(v, (int, float, str, bool))}}) + "\n")
        self.f.flush()

    def finish(self):
        self.f.close()


class _TensorBoard:
    def __init__(self, log_dir: str):
        from torch.utils.tensorboard import SummaryWriter

        self.w = SummaryWriter(log_dir)

    def log(self, data, step):
        for k, v in data.items():
            if isinstance(v, (int, float)):
                self.w.add_scalar(k, v, step)

    def finish(self):
        self.w.close()


class _Wandb:
    def __init__(self, project, name, config, tags=None):
        import wandb

        self.wandb = wandb
        self.run = wandb.init(project=project, name=name, config=config, tags=tags)

    def log(self, data, step):
        self.wandb.log(data, step=step)

    def finish(self):
        self.wandb.finish()


class _MLflow:
    def __init__(self, project, name, config):
        import mlflow

        self.mlflow = mlflow
        mlflow.set_experiment(project)
        mlflow.start_run(run_name=name)
        flat = {}

        def walk(d, pre=""):
            for k, v in d.items():
                if isinstance(v, dict):
                    walk(v, f"{pre}{k}.")
                else:
                    flat[f"{pre}{k}"] = v

        walk(config or {})
        for k, v in list(flat.items())[:400]:
            mlflow.log_param(k, str(v)[:250])

    def log(self, data, step):
        self.mlflow.log_metrics({k.replace("@", "_at_"): float(v) for k, v in data.items() if isinstance(v, (int, float))},
                                step=step)

    def finish(self):
        self.mlflow.end_run()


class Tracking:
    supported = ("console", "jsonl", "tensorboard", "wandb", "mlflow", "swanlab")

    def __init__(self, project_name: str, experiment_name: str, backends: Union[str, List[str]] = "console",
                 config: Optional[Dict[str, Any]] = None, log_dir: str = "/tmp/skyrl-logs", tags=None):
        if isinstance(backends, str):
            backends = [b.strip() for b in backends.split(",") if b.strip()]
        self.loggers: Dict[str, Any] = {}
        for b in backends:
            if b not in self.supported:
                raise ValueError(f"logger '{b}' is not supported; choose from {self.supported}")
            try:
                if b == "console":
                    self.loggers[b] = _Console()
                elif b == "jsonl":
                    self.loggers[b] = _Jsonl(os.path.join(log_dir, f"{experiment_name}.metrics.jsonl"))
                elif b == "tensorboard":
                    self.loggers[b] = _TensorBoard(os.path.join(log_dir, "tensorboard", experiment_name))
                elif b == "wandb":
                    self.loggers[b] = _Wandb(project_name, experiment_name, config, tags)
                elif b == "mlflow":
                    self.loggers[b] = _MLflow(project_name, experiment_name, config)
                elif b == "swanlab":
                    import swanlab

                    swanlab.init(project=project_name, experiment_name=experiment_name, config=config)
                    self.loggers[b] = type("S", (), {"log": staticmethod(lambda d, s: swanlab.log(d, step=s)),
                                                     "finish": staticmethod(swanlab.finish)})()
            except ImportError as e:
                print(f"[tracking] backend '{b}' unavailable ({e}); falling back to console", flush=True)
                self.loggers.setdefault("console", _Console())

    def log(self, data: Dict[str, Any], step: int, commit: bool = True) -> None:
        for lg in self.loggers.values():
            lg.log(data, step)

    def log_exception(self, exc: BaseException) -> None:
        """Surface a crash in every backend before the process dies (reference: main_base.py:322-335)."""
        text = "".join(traceback.format_exception(type(exc), exc, exc.__traceback__))
        for lg in self.loggers.values():
            try:
                lg.log({"exception": text[-4000:]}, 0)
            except Exception:
                pass

    def finish(self) -> None:
        for lg in self.loggers.values():
            try:
                lg.finish()
            except Exception:
                pass

    def __del__(self):
        self.finish()
