"""RL loop on the client, model on a training service.

The reference ships one integration of this shape, ``integrations/arctic_rl`` (trainer.py:65-157, generator.py): its
``ArcticPPOTrainer`` replaces the worker dispatch by calls to an external training server, which owns log-probs, the
surrogate loss, backward and the optimizer, while the client keeps rollouts' reward scoring and the advantage estimate.
The Arctic server and its client library are proprietary, so the service spoken to here is the Tinker-compatible REST
API that this package itself serves (``skyrl_b200/tinker/api.py``) -- any server with those verbs works.
"""

from .client import TrainingServiceClient
from .trainer import RemoteBackendTrainer, RemotePolicyWorker, RemoteSamplerClient, batch_to_datums

__all__ = ["TrainingServiceClient", "RemoteBackendTrainer", "RemotePolicyWorker", "RemoteSamplerClient", "batch_to_datums"]
