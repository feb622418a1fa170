"""Multi-process paths on CPU (gloo, world size 2): tensor-parallel layer logic, sharded optimizer, a 2-rank RL step."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script_args, nproc=2, timeout=900, port=29631):
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port)] + script_args
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_gloo_tp_and_sharded_optimizer():
    p = _run([os.path.join(ROOT, "tests", "mp", "cpu_checks.py")])
    assert p.returncode == 0 and "CPU_CHECKS_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_two_rank_rl_step():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-qwen2-d128",
              "--prompts-per-gpu", "1"], port=29632)
    assert p.returncode == 0 and '"n_gpus": 2' in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_two_rank_tensor_parallel_rl_step():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-llama",
              "--prompts-per-gpu", "1", "--tp", "2"], port=29633)
    assert p.returncode == 0 and "x tp2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_two_rank_sequence_parallel_rl_step():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-llama",
              "--prompts-per-gpu", "1", "--sp", "2"], port=29634)
    assert p.returncode == 0 and "x sp2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_two_rank_expert_parallel_rl_step():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-moe",
              "--prompts-per-gpu", "1", "--ep", "2"], port=29635)
    assert p.returncode == 0 and "x ep2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_two_rank_pipeline_parallel_rl_step():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-llama",
              "--prompts-per-gpu", "1", "--pp", "2"], port=29636)
    assert p.returncode == 0 and "x pp2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


import pytest  # noqa: E402


@pytest.mark.parametrize("mode,port", [("tp", 29641), ("sp", 29642), ("ep", 29643), ("pp", 29644), ("tpv", 29648),
                                       ("critic_tp", 29649), ("critic_sp", 29650), ("cp", 29663),
                                       ("cp_megatron", 29664), ("critic_cp", 29665), ("pp_mb1", 29671)])
def test_gloo_worker_update_matches_single_rank(mode, port):
    """forward_backward + optim_step through the worker under each model-parallel strategy: full parameters equal a
    single-rank update on the same data, group replicas are bit-identical, one optimizer step per RL step."""
    p = _run([os.path.join(ROOT, "tests", "mp", "worker_parity.py"), mode], port=port)
    assert p.returncode == 0 and f"WORKER_PARITY_OK mode={mode}" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_engine_tensor_parallel_matches_unsharded():
    p = _run([os.path.join(ROOT, "tests", "mp", "engine_tp_check.py")], port=29645)
    assert p.returncode == 0 and "ENGINE_TP_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_rl_step_with_tensor_parallel_engine():
    for extra, port in ((["--engine-tp", "2"], 29646), (["--tp", "2", "--engine-tp", "2"], 29647)):
        p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-llama",
                  "--prompts-per-gpu", "1", *extra], port=port)
        assert p.returncode == 0 and '"n_gpus": 2' in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_hybrid_sharded_optimizer_four_ranks():
    p = _run([os.path.join(ROOT, "tests", "mp", "hsdp_check.py")], nproc=4, port=29651)
    assert p.returncode == 0 and "HSDP_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.parametrize("nproc,port", [(2, 29661), (4, 29662)])
def test_gloo_token_balancing_keeps_the_update_and_evens_the_loads(nproc, port):
    p = _run([os.path.join(ROOT, "tests", "mp", "balance_check.py")], nproc=nproc, port=port)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert f"BALANCE_OK world={nproc}" in p.stdout


@pytest.mark.parametrize("nproc,port", [(2, 29666), (3, 29667)])
def test_gloo_context_parallel_model_matches_plain_model(nproc, port):
    """Key/value all-gather context parallelism: log-probs and summed weight gradients equal the plain model's, also
    at a degree (3) that does not divide the two key/value heads."""
    p = _run([os.path.join(ROOT, "tests", "mp", "cp_check.py")], nproc=nproc, port=port)
    assert p.returncode == 0 and f"CP_MODEL_OK world={nproc}" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_gloo_two_rank_context_parallel_rl_step():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-llama",
              "--prompts-per-gpu", "1", "--sp", "2", "--sp-backend", "context"], port=29668)
    assert p.returncode == 0 and '"n_gpus": 2' in p.stdout and "context parallel" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
