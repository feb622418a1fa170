"""Lock-step driver for a tensor-parallel generation engine: one request stream, ``tp`` identical engine replicas.

Every rank of an engine's tensor-parallel group runs its own ``LLMEngine`` (scheduler, block tables, decode state)
over its shard of the weights and of the KV cache; the ranks never exchange tokens because their arithmetic is
bit-identical (``engine/tp_model.py``).  What they must share is the *order of operations*: which requests are added
before which step, when the engine pauses, when weights change.  The group's leader (tp rank 0) owns the request
stream -- generators, environments and clients talk to it alone -- and before each step it broadcasts the operations
queued since the previous step over the group's host channel (gloo); every rank applies them and steps.  Followers
sit in ``follow()`` while the leader generates.  This is the role vLLM's driver / worker split plays for the
reference's ``tensor_parallel_size > 1`` engines (inference_servers/utils.py:89-100), without an RPC layer: the
follower is the same SPMD process that trains.
"""

from __future__ import annotations

from typing import Any, List, Optional, Sequence

import torch.distributed as dist

from .llm_engine import LLMEngine, RequestOutput, SamplingParams

_FORWARDED = ("abort_request", "pause", "resume", "reset_prefix_cache", "sleep", "wake_up", "on_weights_updated")


class LockstepEngine:
    def __init__(self, engine: LLMEngine, group, leader_global_rank: int):
        self.engine = engine
        self.group = group
        self.leader = leader_global_rank
        self.is_leader = dist.get_rank() == leader_global_rank
        self._ops: List[tuple] = []

    # ------------------------------------------------------------------ pass-through state
    def __getattr__(self, name: str) -> Any:  # cfg, stats, weight_version, paused, asleep, model, metrics(), ...
        return getattr(self.engine, name)

    # ------------------------------------------------------------------ leader side
    def _queue(self, op: tuple) -> None:
        assert self.is_leader, "only the leader of a tensor-parallel engine group accepts requests"
        self._ops.append(op)

    def add_request(self, request_id: str, prompt_token_ids: Sequence[int], params: SamplingParams,
                    cache_salt: Optional[str] = None) -> None:
        self._queue(("add", request_id, [int(t) for t in prompt_token_ids], params, cache_salt))

    def _exchange(self, stop: bool = False) -> None:
        box = [(self._ops, stop)]
        dist.broadcast_object_list(box, src=self.leader, group=self.group)
        self._ops = []
        self._apply(box[0][0])

    def _apply(self, ops: List[tuple]) -> None:
        for op in ops:
            if op[0] == "add":
                self.engine.add_request(op[1], op[2], op[3], op[4])
            else:
                getattr(self.engine, op[1])(*op[2], **op[3])

    def step(self) -> List[RequestOutput]:
        self._exchange()
        return self.engine.step()

    def has_unfinished(self) -> bool:
        return bool(self._ops) or self.engine.has_unfinished()

    def generate(self, prompts, params, request_ids=None, cache_salt=None) -> List[RequestOutput]:
        if isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        rids = list(request_ids) if request_ids is not None else [f"lgen-{id(self)}-{self.engine._next_sid}-{i}"
                                                                   for i in range(len(prompts))]
        for rid, p, sp in zip(rids, prompts, params):
            self.add_request(rid, p, sp, cache_salt)
        got = {}
        while set(rids) - set(got):
            for o in self.step():
                got[o.request_id] = o
        return [got[r] for r in rids]

    def end_generation(self) -> None:
        """Leader: release the followers from ``follow()`` (also flushes control operations queued after the last step)."""
        self._exchange(stop=True)

    # ------------------------------------------------------------------ follower side
    def follow(self) -> None:
        """Follower: mirror the leader's operations and steps until it calls ``end_generation``."""
        assert not self.is_leader
        while True:
            box = [None]
            dist.broadcast_object_list(box, src=self.leader, group=self.group)
            ops, stop = box[0]
            self._apply(ops)
            if stop:
                return
            self.engine.step()


def _forward(name: str):
    """Control operations.  While the leader has requests in flight they are queued and reach every rank with the next
    step's broadcast (the stepping loop keeps calling ``step`` while paused, see ``lockstep`` below); between
    generation phases every rank runs the same controller code, so each applies the call to its own engine."""

    def call(self, *args, **kwargs):
        if self.is_leader and (self._ops or self.engine.has_unfinished()):
            self._queue(("call", name, args, kwargs))
            return [] if name == "pause" else None
        return getattr(self.engine, name)(*args, **kwargs)

    return call


for _n in _FORWARDED:
    setattr(LockstepEngine, _n, _forward(_n))

LockstepEngine.lockstep = True  # stepping loops must keep calling step() while the engine is paused
