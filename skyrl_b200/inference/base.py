"""Inference-engine interface shared by the in-process client, the HTTP client and test fakes.

Method set and I/O dictionaries follow the reference
(skyrl/backends/skyrl_train/inference_servers/base.py:27-171): token-in / token-out ``generate``,
OpenAI-style ``chat_completion`` / ``completion``, and the control plane (``pause`` / ``resume`` /
``sleep`` / ``wake_up`` / ``reset_prefix_cache`` / weight-update verbs / ``finish_session``).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, List, Optional, TypedDict

ConversationType = List[Dict[str, Any]]


class InferenceEngineInput(TypedDict, total=False):
    prompts: Optional[List[ConversationType]]
    prompt_token_ids: Optional[List[List[int]]]
    sampling_params: Optional[Dict[str, Any]]
    session_ids: Optional[List[Any]]
    mm_features: Optional[List[Any]]
    cache_salt: Optional[str]


class InferenceEngineOutput(TypedDict, total=False):
    responses: List[str]
    response_ids: List[List[int]]
    stop_reasons: List[str]
    response_logprobs: Optional[List[List[float]]]
    prompt_logprobs: Optional[List[List[float]]]
    rollout_expert_indices: Optional[List[Any]]
    weight_versions: Optional[List[int]]


class InferenceEngineInterface(ABC):
    @abstractmethod
    async def generate(self, input_batch: InferenceEngineInput) -> InferenceEngineOutput: ...

    async def chat_completion(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        raise NotImplementedError

    async def completion(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        raise NotImplementedError

    async def render(self, request_payload: Dict[str, Any]) -> Dict[str, Any]:
        raise NotImplementedError

    @abstractmethod
    async def pause(self, mode: str = "keep", clear_cache: bool = False) -> None: ...

    @abstractmethod
    async def resume(self) -> None: ...

    @abstractmethod
    async def sleep(self, level: int = 2, tags: Optional[List[str]] = None) -> None: ...

    @abstractmethod
    async def wake_up(self, tags: Optional[List[str]] = None) -> None: ...

    @abstractmethod
    async def reset_prefix_cache(self, reset_running_requests: bool = False) -> None: ...

    async def init_weight_update_communicator(self, init_info: Any) -> None:
        return None

    async def update_named_weights(self, request: Any) -> None:
        raise NotImplementedError

    async def finish_session(self, session_id: Any) -> None:
        return None

    async def teardown(self) -> None:
        return None

    def get_world_size(self) -> int:
        return 1

    def tp_size(self) -> int:
        return 1

    def pp_size(self) -> int:
        return 1

    def dp_size(self) -> int:
        return 1
