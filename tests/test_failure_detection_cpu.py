"""Failure detection on the host only: a rank that exits takes the job down through the launcher, a rank that never
joins a collective is reported by the process-group timeout, damaged checkpoints are refused with a clear error, the
pointer file never runs ahead of the data."""
import os
import subprocess
import sys
import textwrap
import time

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _write(tmp_path, name, body):
    p = tmp_path / name
    p.write_text(textwrap.dedent(body))
    return str(p)


def test_launcher_tears_down_survivors_when_a_rank_dies(tmp_path):
    script = _write(tmp_path, "job.py", """
        import os, sys, time
        r = int(os.environ["RANK"])
        open(os.path.join(os.path.dirname(__file__), f"started_{r}"), "w").close()
        if r == 1:
            time.sleep(0.5)
            sys.exit(7)
        time.sleep(120)   # a healthy rank that would otherwise keep the job alive
    """)
    t0 = time.time()
    p = subprocess.run([sys.executable, "-m", "skyrl_b200.launch", "--nproc-per-node", "3", "--no-numa-pin", script],
                       cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES=""), capture_output=True,
                       text=True, timeout=90)
    assert p.returncode == 7, p.stderr[-2000:]
    assert time.time() - t0 < 60  # survivors were terminated, not waited for
    assert "rank 1 exited with 7" in p.stderr
    assert all(os.path.exists(tmp_path / f"started_{r}") for r in range(3))


def test_launcher_environment_and_success(tmp_path):
    script = _write(tmp_path, "env.py", """
        import os
        assert os.environ["MASTER_ADDR"] == "127.0.0.1" and int(os.environ["WORLD_SIZE"]) == 2
        assert os.environ["LOCAL_RANK"] == os.environ["RANK"]
        print("rank", os.environ["RANK"], "ok")
    """)
    p = subprocess.run([sys.executable, "-m", "skyrl_b200.launch", "--nproc-per-node", "2", "--no-numa-pin", script],
                       cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES=""), capture_output=True,
                       text=True, timeout=60)
    assert p.returncode == 0 and p.stdout.count("ok") == 2


def test_missing_rank_surfaces_as_collective_timeout(tmp_path):
    script = _write(tmp_path, "hang.py", """
        import datetime, os, sys, time
        import torch, torch.distributed as dist
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
        r = dist.get_rank()
        dist.barrier()
        if r == 1:
            time.sleep(30)        # never joins the next collective in time
            sys.exit(0)
        t = torch.ones(1)
        try:
            dist.all_reduce(t)
            print("UNEXPECTED_SUCCESS")
        except Exception as e:
            print("DETECTED", type(e).__name__)
            sys.exit(3)
    """)
    p = subprocess.run([sys.executable, "-m", "skyrl_b200.launch", "--nproc-per-node", "2", "--no-numa-pin", script],
                       cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES=""), capture_output=True,
                       text=True, timeout=120)
    assert "DETECTED" in p.stdout and "UNEXPECTED_SUCCESS" not in p.stdout
    assert p.returncode == 3


def test_truncated_or_mismatched_checkpoint_is_refused(tmp_path):
    from skyrl_b200.config.config import SkyRLTrainConfig
    from skyrl_b200.parallel.dist import get_env
    from skyrl_b200.train import utils as tutils
    from skyrl_b200.workers.worker import PolicyWorker

    cfg = SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model.path=tiny-llama", "trainer.bf16=false"])
    w = PolicyWorker(cfg.trainer, model_path="tiny-llama", env=get_env(), seed=0)
    d = str(tmp_path / "global_step_3" / "policy")
    w.save_checkpoint(d, tag="3")
    f = os.path.join(d, "model_world_size_1_rank_0.pt")
    blob = open(f, "rb").read()
    open(f, "wb").write(blob[: len(blob) // 2])  # torn write
    with pytest.raises(Exception):
        w.load_checkpoint(d)
    os.remove(f)
    with pytest.raises(FileNotFoundError) as e:
        w.load_checkpoint(d)
    assert "world size" in str(e.value)
    # the latest-pointer is written last and must point at an existing directory
    tutils.write_latest(str(tmp_path), 9)
    cfg.trainer.ckpt_path, cfg.trainer.resume_mode = str(tmp_path), "latest"
    with pytest.raises(FileNotFoundError):
        tutils.resolve_resume_path(cfg.trainer)


def test_bounded_wait_status_codes_are_documented():
    """Every device wait site writes a distinct non-zero code; the host API reads and clears it (no GPU needed to check
    that the codes used in the sources are unique per site)."""
    import glob
    import re

    codes = []
    for f in glob.glob(os.path.join(ROOT, "skyrl_b200", "csrc", "*.cu")):
        src = open(f).read()
        codes += [(os.path.basename(f), c) for c in re.findall(r"mbar_wait\([^;]*?,\s*(0x[0-9a-fA-F]+)\)", src)]
    assert len(codes) > 20
    per_file = {}
    for f, c in codes:
        per_file.setdefault(f, []).append(c)
    assert all(int(c, 16) != 0 for _, c in codes)
