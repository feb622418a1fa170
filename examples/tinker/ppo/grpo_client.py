"""RL loop written against the Tinker-compatible REST API only: the client owns prompts, rewards and advantages; the
service owns sampling, log-probs, the clipped objective and the optimizer.  Start the service with

    python -m skyrl_b200.tinker.api --base-model qwen2.5-1.5b --port 8000

then ``python examples/tinker/ppo/grpo_client.py http://127.0.0.1:8000``.  The reward here is a toy (fraction of even
token ids in the response) so that the script needs no dataset; swap ``reward_fn`` for your own.
Counterpart in the reference: examples/tinker/ppo (a PPO client on the Tinker SDK).
"""

import sys
from typing import Callable, Dict, List

import requests


def http_caller(url: str) -> Callable[[str, Dict], Dict]:
    def call(path: str, body: Dict) -> Dict:
        while True:
            r = requests.post(url + path, json=body, timeout=600)
            if path.endswith("retrieve_future") and r.status_code == 408:
                continue  # long poll ran out: ask again
            r.raise_for_status()
            return r.json()

    return call


def reward_fn(prompt: List[int], response: List[int]) -> float:
    return sum(1 for t in response if t % 2 == 0) / max(1, len(response))


def grpo_datum(prompt: List[int], response: List[int], logprobs: List[float], advantage: float) -> Dict:
    """One trajectory as a Tinker datum: inputs are all tokens but the last, targets all but the first; only response
    positions carry weight, rollout log-probs and the (sequence-level) advantage."""
    tokens = prompt + response
    n, p = len(tokens) - 1, len(prompt) - 1
    col = lambda vals, dt: {"data": vals, "dtype": dt, "shape": [n]}  # noqa: E731
    return {"model_input": {"chunks": [{"type": "encoded_text", "tokens": tokens[:-1]}]},
            "loss_fn_inputs": {"target_tokens": col(tokens[1:], "int64"),
                               "weights": col([0.0] * p + [1.0] * len(response), "float32"),
                               "logprobs": col([0.0] * p + list(logprobs), "float32"),
                               "advantages": col([0.0] * p + [advantage] * len(response), "float32")}}


def run(call: Callable[[str, Dict], Dict], base_model: str, prompts: List[List[int]], steps: int = 3, group: int = 4,
        max_tokens: int = 16, lr: float = 1e-5, lora_rank: int = 0) -> List[float]:
    wait = lambda fut: call("/api/v1/retrieve_future", {"request_id": fut["request_id"]})  # noqa: E731
    sid = call("/api/v1/create_session", {"tags": ["grpo-example"], "sdk_version": "example"})["session_id"]
    m = call("/api/v1/create_model", {"session_id": sid, "base_model": base_model, "lora_config": {"rank": lora_rank}})
    wait(m)
    mid, seq, mean_rewards = m["model_id"], 0, []
    for step in range(steps):
        # 1. publish the current weights and sample a group per prompt
        ss = wait(call("/api/v1/save_weights_for_sampler", {"model_id": mid, "sampling_session_seq_id": step}))
        futs = [call("/api/v1/asample", {"sampling_session_id": ss["sampling_session_id"], "num_samples": group,
                                          "prompt": {"chunks": [{"tokens": p}]},
                                          "sampling_params": {"max_tokens": max_tokens, "temperature": 1.0}}) for p in prompts]
        data, rewards = [], []
        for p, fut in zip(prompts, futs):
            seqs = wait(fut)["sequences"]
            rs = [reward_fn(p, s["tokens"]) for s in seqs]
            mean = sum(rs) / len(rs)
            std = (sum((r - mean) ** 2 for r in rs) / len(rs)) ** 0.5
            rewards += rs
            for s, r in zip(seqs, rs):  # 2. group-relative advantages
                if s["tokens"]:
                    data.append(grpo_datum(p, s["tokens"], s["logprobs"], (r - mean) / (std + 1e-6)))
        # 3. clipped policy-gradient step on the service
        fb = call("/api/v1/forward_backward", {"model_id": mid, "seq_id": seq,
                                               "forward_backward_input": {"data": data, "loss_fn": "ppo"}})
        op = call("/api/v1/optim_step", {"model_id": mid, "seq_id": seq + 1, "adam_params": {"learning_rate": lr}})
        seq += 2
        fbm, opm = wait(fb)["metrics"], wait(op)["metrics"]
        mean_rewards.append(sum(rewards) / len(rewards))
        print(f"step {step}: mean reward {mean_rewards[-1]:.3f}, {len(data)} trajectories, "
              f"loss {fbm.get('loss:sum', float('nan')):.4f}, grad norm {opm.get('grad_norm', float('nan')):.4f}")
    return mean_rewards


if __name__ == "__main__":
    url = sys.argv[1] if len(sys.argv) > 1 else "http://127.0.0.1:8000"
    base = sys.argv[2] if len(sys.argv) > 2 else "qwen2.5-1.5b"
    run(http_caller(url), base, [[100 + 7 * i, 200 + i, 300] for i in range(8)])
