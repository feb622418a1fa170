"""Multi-GPU checks, each run as torchrun child processes on 2 GPUs (skipped on single-GPU boxes)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script_args, nproc=2, timeout=600, port=29617):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port)] + script_args
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_collectives_match_nccl():
    p = _run([os.path.join(ROOT, "tests", "mp", "peer_checks.py")])
    assert p.returncode == 0 and "PEER_CHECKS_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_bench_two_gpus_tiny():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-qwen2-d128",
              "--prompts-per-gpu", "4"], port=29618)
    assert p.returncode == 0 and '"n_gpus": 2' in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_fused_gemm_collectives():
    p = _run([os.path.join(ROOT, "tests", "mp", "tp_checks.py")], port=29619)
    assert p.returncode == 0 and "TP_CHECKS" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_bench_two_gpus_tensor_parallel_tiny():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-qwen2-tp",
              "--prompts-per-gpu", "4", "--tp", "2"], port=29620)
    assert p.returncode == 0 and "x tp2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_bench_two_gpus_sequence_parallel_and_expert_parallel_tiny():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-qwen2-tp",
              "--prompts-per-gpu", "4", "--sp", "2"], port=29621)
    assert p.returncode == 0 and "x sp2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-moe",
              "--prompts-per-gpu", "4", "--ep", "2"], port=29622)
    assert p.returncode == 0 and "x ep2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_bench_two_gpus_pipeline_parallel_tiny():
    p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-qwen2-tp",
              "--prompts-per-gpu", "4", "--pp", "2"], port=29623)
    assert p.returncode == 0 and "x pp2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_engine_tensor_parallel_matches_unsharded_engine():
    """TP=2 engine (all-reduce in the o-proj / down-proj epilogues, eager and CUDA-graph decode) vs TP=1."""
    p = _run([os.path.join(ROOT, "tests", "mp", "engine_tp_check.py")], port=29624)
    assert p.returncode == 0 and "ENGINE_TP_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_weight_sync_relayout_kernel_is_bit_exact():
    p = _run([os.path.join(ROOT, "tests", "mp", "relayout_check.py")], port=29625)
    assert p.returncode == 0 and "RELAYOUT_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_bench_two_gpus_tensor_parallel_engine_tiny():
    """RL step with a TP=2 rollout engine, under a data-parallel and under a tensor-parallel trainer."""
    for extra, port in ((["--engine-tp", "2"], 29626), (["--tp", "2", "--engine-tp", "2"], 29627)):
        p = _run([os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "1", "--model", "tiny-qwen2-tp",
                  "--prompts-per-gpu", "4", *extra], port=port)
        assert p.returncode == 0 and '"device_status": 0' in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_gradient_reduce_scatter_behind_backward_matches_one_shot():
    p = _run([os.path.join(ROOT, "tests", "mp", "overlap_check.py")], port=29628)
    assert p.returncode == 0 and "OVERLAP_REDUCE_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
