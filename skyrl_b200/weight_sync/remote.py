"""Weight sync between a trainer and stand-alone rollout servers (different processes, possibly different machines).

Trainer side ``RemoteWeightSync``: pause the servers (in-flight requests are kept), publish the new weights, tell every
server to load them, resume -- the choreography of the reference's ``save_weights_for_sampler``
(skyrl/backends/skyrl_train/workers/worker_dispatch.py:629-711) with generation always resumed, also after a failure
(:702-707).  Two transports:

* ``delta``  : XOR deltas against the last publication in a shared directory (``weight_sync/delta.py``); servers replay
  them into their local copy and load the result (reference: delta_strategy.py + delta_checkpoint.py).
* ``path``   : a full HF-safetensors export that the servers read (simple, for small models and tests).
* ``peer``   : servers on GPUs of the same NVSwitch domain export their parameter buffer through a CUDA IPC handle
  (``/init_weight_transfer_engine``); every trainer rank maps the buffers once and pushes the blocks it owns straight
  into them with the re-layout kernel (``weight_sync/relayout.py``) between ``pause(keep)`` and ``resume``.  No rank-0
  funnel, no files, no per-sync handles (reference: NCCL broadcast from trainer rank 0, broadcast_strategy.py:131-183).

Server side ``make_weight_loader(model, engine, ...)`` returns the callable that ``inference.server.build_app`` invokes
for the weight verbs.
"""

from __future__ import annotations

import os
import tempfile
from typing import Any, Callable, Dict, Optional

import torch

from .delta import DeltaPublisher, LocalCheckpointStore


def _named_state(model) -> Dict[str, torch.Tensor]:
    return {name: prm.detach() for name, prm in model.named_flat_views()}


def make_weight_loader(model, engine=None, sync_dir: Optional[str] = None, local_dir: Optional[str] = None,
                       ipc_handle: Optional[str] = None) -> Callable:
    """``loader(kind, payload)`` for ``/init_weight_transfer_engine``, ``/fetch_weights``, ``/update_weights``.
    ``ipc_handle``: CUDA IPC handle (hex) of the model's flat parameter buffer when it was allocated for export."""
    store: Dict[str, Any] = {"delta": None}

    def _after_load():
        if engine is not None:
            engine.on_weights_updated(clear_kv=True)

    @torch.no_grad()
    def loader(kind: str, payload: Dict[str, Any]) -> Dict[str, Any]:
        if kind == "init":
            import socket

            info = {"ready": True, "host": socket.gethostname(), "numel": int(model.flat_params.numel()),
                    "dtype": str(model.flat_params.dtype).replace("torch.", ""),
                    "device_index": model.flat_params.device.index}
            if ipc_handle is not None:
                info["ipc_handle"] = ipc_handle
            return info
        if kind == "fetch_weights":
            sd = payload.get("sync_dir") or sync_dir
            if sd is None:
                raise ValueError("fetch_weights needs a sync_dir")
            if store["delta"] is None or store["delta"].sync_dir != sd:
                ld = local_dir or os.path.join(tempfile.gettempdir(), f"skyrl_b200_delta_{os.getpid()}")
                store["delta"] = LocalCheckpointStore(sd, ld)
            v = store["delta"].fetch(int(payload["version"]))
            state = store["delta"].state_dict()
            for name, prm in model.named_flat_views():
                prm.copy_(state[name].to(prm.dtype))
            _after_load()
            return {"loaded_version": v}
        if kind == "update_weights":
            from ..models import hf_io

            path = payload.get("load_path")
            if not path:
                raise ValueError("update_weights over HTTP needs load_path (packed tensors travel by peer push or broadcast)")
            hf_io.load_hf_weights(model, path)
            _after_load()
            return {"loaded_path": path}
        if kind in ("start_weight_update", "finish_weight_update"):
            if kind == "finish_weight_update":
                _after_load()
            return {}
        raise ValueError(f"unsupported weight verb '{kind}'")

    return loader


class RemoteWeightSync:
    def __init__(self, client, model, transport: str = "delta", sync_dir: Optional[str] = None, is_main: bool = True,
                 pause_mode: str = "keep", peer_plan: Optional[Callable] = None):
        """``peer_plan(dest_pointers) -> RelayoutPush`` builds this rank's push plan once the servers' buffers are
        mapped (``peer`` transport only; every trainer rank takes part, rank 0 alone drives pause / resume)."""
        if transport not in ("delta", "path", "peer"):
            raise ValueError(f"unknown remote weight transport '{transport}'")
        self.peer_plan, self._push = peer_plan, None
        self.last_push_ms: Optional[float] = None
        self.client, self.model, self.transport, self.is_main, self.pause_mode = client, model, transport, is_main, pause_mode
        self.sync_dir = sync_dir or os.path.join(tempfile.gettempdir(), f"skyrl_b200_sync_{os.getpid()}")
        self.publisher = DeltaPublisher(self.sync_dir) if (transport == "delta" and is_main) else None
        self.version = 0

    async def sync(self) -> int:
        """Publish the model's current weights and make every server load them. Returns the published version."""
        if self.transport == "peer":
            return await self._sync_peer()
        if not self.is_main:
            return self.version
        await self.client.pause(self.pause_mode)
        try:
            if self.transport == "delta":
                state = _named_state(self.model)
                if not self.publisher.snapshot:
                    self.publisher.publish_base(state)
                    self.version = 0
                else:
                    self.publisher.publish(state)
                    self.version = self.publisher.version
                await self.client.fetch_weights({"sync_dir": self.sync_dir, "version": self.version})
            else:
                from ..models import hf_io

                self.version += 1
                path = os.path.join(self.sync_dir, f"export-{self.version:08d}")
                hf_io.save_hf_model(self.model, path)
                await self.client.update_weights({"load_path": path}) if hasattr(self.client, "update_weights") else \
                    await self.client._fanout("/update_weights", {"load_path": path})
        finally:
            await self.client.resume()  # generation always continues, also when the transfer failed
        return self.version

    async def _sync_peer(self) -> int:
        import torch.distributed as dist

        from ..parallel.peer import ipc_open

        multi = dist.is_initialized() and dist.get_world_size() > 1
        if self._push is None:
            infos = await self.client._fanout("/init_weight_transfer_engine", {"transport": "peer"})
            missing = [i for i, x in enumerate(infos) if not (isinstance(x, dict) and x.get("ipc_handle"))]
            if missing:
                raise RuntimeError(f"rollout servers {missing} did not export a parameter buffer for peer weight sync")
            self._push = self.peer_plan([ipc_open(x["ipc_handle"]) for x in infos])
        if self.is_main:
            await self.client.pause(self.pause_mode)
        try:
            if multi:
                dist.barrier()  # no rank writes before every server has stopped reading its weights
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            self._push.run()
            ev1.record()
            ev1.synchronize()  # this rank's stores have reached the engines' memory
            self.last_push_ms = ev0.elapsed_time(ev1)
            if multi:
                dist.barrier()
            self.version += 1
            if self.is_main:
                await self.client.collective_rpc("finish_weight_update")
        finally:
            if self.is_main:
                await self.client.resume()
        return self.version
