"""Dispatchers: how the (instance x trajectory) grid of agent episodes is scheduled.

Reference (peripheral package): skyrl-agent/skyrl_agent/dispatcher/dispatchers.py (a registry with ``async_batch``
and ``async_pipeline``).  ``async_batch`` runs every episode start to finish under one concurrency limit;
``async_pipeline`` connects the three stages (initialise, run, evaluate) by queues with their own limits, so a slow
evaluation (a test suite, a judge) does not hold a generation slot.
"""

from __future__ import annotations

import asyncio
from typing import Any, Awaitable, Callable, Dict, List, Tuple

Stage = Callable[[int, int], Awaitable[Any]]  # (instance index, trajectory index)

DISPATCHER_REGISTRY: Dict[str, Callable[..., Awaitable[None]]] = {}


def register_dispatcher(name: str):
    def deco(fn):
        DISPATCHER_REGISTRY[name] = fn
        return fn

    return deco


def _grid(n_instances: int, n_trajectories: int) -> List[Tuple[int, int]]:
    # trajectory-major: the first samples of all instances start before anyone's second sample
    return [(i, t) for t in range(n_trajectories) for i in range(n_instances)]


@register_dispatcher("async_batch")
async def async_batch(cfg: Dict[str, Any], n_instances: int, n_trajectories: int, init: Stage, run: Stage, evaluate: Stage) -> None:
    sem = asyncio.Semaphore(max(1, int(cfg.get("max_parallel_agents", 64))))

    async def one(i: int, t: int):
        async with sem:
            await init(i, t)
            await run(i, t)
            await evaluate(i, t)

    await asyncio.gather(*[one(i, t) for i, t in _grid(n_instances, n_trajectories)])


@register_dispatcher("async_pipeline")
async def async_pipeline(cfg: Dict[str, Any], n_instances: int, n_trajectories: int, init: Stage, run: Stage, evaluate: Stage) -> None:
    total = n_instances * n_trajectories
    n_run = max(1, min(total, int(cfg.get("max_parallel_agents", 64))))
    n_eval = max(1, min(total, int(cfg.get("max_eval_parallel_agents", n_run))))
    n_init = max(1, min(total, int(cfg.get("max_init_parallel_agents", n_run))))
    q_init: asyncio.Queue = asyncio.Queue()
    q_run: asyncio.Queue = asyncio.Queue()
    q_eval: asyncio.Queue = asyncio.Queue()
    errors: List[BaseException] = []
    for item in _grid(n_instances, n_trajectories):
        q_init.put_nowait(item)

    async def worker(src: asyncio.Queue, dst, stage: Stage):
        while True:
            item = await src.get()
            try:
                await stage(*item)
            except BaseException as e:  # noqa: BLE001 - reported after the pipeline drained
                errors.append(e)
            finally:
                if dst is not None:
                    dst.put_nowait(item)
                src.task_done()

    workers = ([asyncio.create_task(worker(q_init, q_run, init)) for _ in range(n_init)]
               + [asyncio.create_task(worker(q_run, q_eval, run)) for _ in range(n_run)]
               + [asyncio.create_task(worker(q_eval, None, evaluate)) for _ in range(n_eval)])
    try:
        await q_init.join()
        await q_run.join()
        await q_eval.join()
    finally:
        for w in workers:
            w.cancel()
        await asyncio.gather(*workers, return_exceptions=True)
    if errors:
        raise errors[0]
