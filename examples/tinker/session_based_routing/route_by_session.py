"""Multi-turn sampling that keeps every conversation on one rollout server, so its KV prefix stays cached there.

Several servers (``examples/serve/run_serve.sh``) sit behind the session-affine router; a request that carries an
``X-Session-ID`` header always reaches the same server (rendezvous hashing over the healthy ones), requests without
one are spread.  This script drives ``n`` conversations of ``turns`` turns each through the router and prints which
server answered what, using the stack's own client.
Counterpart in the reference: examples/tinker/session_based_routing.
"""

import asyncio
import sys
from collections import defaultdict
from typing import Dict, List

from skyrl_b200.inference.remote_client import RemoteInferenceClient
from skyrl_b200.inference.router import SessionRouter


async def converse(client: RemoteInferenceClient, sessions: int = 4, turns: int = 3, max_tokens: int = 8) -> Dict[str, List[List[int]]]:
    out: Dict[str, List[List[int]]] = defaultdict(list)

    async def one(i: int) -> None:
        sid = f"conv-{i}"
        ctx = [100 + i, 200, 300]
        for _ in range(turns):
            r = await client.generate({"prompt_token_ids": [ctx], "session_ids": [sid],
                                       "sampling_params": {"max_generate_length": max_tokens, "temperature": 0.0}})
            out[sid].append(r["response_ids"][0])
            ctx = ctx + r["response_ids"][0] + [400 + i]  # the model's turn, then a new "user" token
        await client.finish_session(sid)

    await asyncio.gather(*[one(i) for i in range(sessions)])
    return dict(out)


if __name__ == "__main__":
    urls = sys.argv[1:] or ["http://127.0.0.1:8001", "http://127.0.0.1:8002"]
    router = SessionRouter(urls)
    for i in range(4):
        print(f"conv-{i} -> {router.pick(f'conv-{i}')}")

    async def main():
        async with RemoteInferenceClient(urls) as client:
            for sid, turns in (await converse(client)).items():
                print(sid, [len(t) for t in turns])

    asyncio.run(main())
