"""Minimal client of the Tinker-compatible service (start it with
``python -m skyrl_b200.tinker.api --base-model qwen2.5-1.5b --port 8000``): supervised steps, then sampling."""

import sys

import requests

URL = sys.argv[1] if len(sys.argv) > 1 else "http://127.0.0.1:8000"


def call(path, body):
    r = requests.post(URL + path, json=body, timeout=600)
    r.raise_for_status()
    return r.json()


def wait(fut):
    while True:
        r = requests.post(URL + "/api/v1/retrieve_future", json={"request_id": fut["request_id"]}, timeout=600)
        if r.status_code == 408:
            continue
        r.raise_for_status()
        return r.json()


def datum(tokens):
    n = len(tokens) - 1
    return {"model_input": {"chunks": [{"type": "encoded_text", "tokens": tokens[:-1]}]},
            "loss_fn_inputs": {"target_tokens": {"data": tokens[1:], "dtype": "int64", "shape": [n]},
                               "weights": {"data": [1.0] * n, "dtype": "float32", "shape": [n]}}}


if __name__ == "__main__":
    sid = call("/api/v1/create_session", {"tags": ["example"], "sdk_version": "example"})["session_id"]
    m = call("/api/v1/create_model", {"session_id": sid, "base_model": "qwen2.5-1.5b", "lora_config": {"rank": 0}})
    wait(m)
    data = [datum([100 + i, 200, 300, 400, 500]) for i in range(8)]
    for step in range(3):
        fb = call("/api/v1/forward_backward", {"model_id": m["model_id"], "forward_backward_input": {"data": data, "loss_fn": "cross_entropy"}})
        op = call("/api/v1/optim_step", {"model_id": m["model_id"], "adam_params": {"learning_rate": 1e-5}})
        print("step", step, wait(fb)["metrics"], wait(op)["metrics"])
    ss = wait(call("/api/v1/save_weights_for_sampler", {"model_id": m["model_id"], "sampling_session_seq_id": 0}))
    out = wait(call("/api/v1/asample", {"sampling_session_id": ss["sampling_session_id"], "num_samples": 2,
                                         "prompt": {"chunks": [{"tokens": [100, 200]}]},
                                         "sampling_params": {"max_tokens": 16, "temperature": 1.0}}))
    print([s["tokens"] for s in out["sequences"]])
