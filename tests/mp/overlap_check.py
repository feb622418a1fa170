"""Run under torchrun on 2 GPUs: the gradient reduce-scatter that starts behind the last micro-batch's backward pass
(layer by layer, on a side stream) gives the same update as the one-shot reduce-scatter after backward."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.config.config import SkyRLTrainConfig  # noqa: E402
from skyrl_b200.ops import _lib  # noqa: E402
from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.parallel.peer import PeerContext  # noqa: E402
from skyrl_b200.train.batch import TrainingInputBatch  # noqa: E402
from skyrl_b200.workers.worker import PolicyWorker  # noqa: E402


def cfg(overlap: bool):
    return SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-qwen2-d128", "trainer.micro_train_batch_size_per_gpu=2",
        "trainer.max_tokens_per_microbatch=0", "trainer.algorithm.use_kl_loss=false", "trainer.gradient_checkpointing=false",
        "trainer.policy.optimizer_config.lr=1e-3", "trainer.policy.optimizer_config.max_grad_norm=1000000.0",
        f"trainer.b200.overlap_grad_reduce={'true' if overlap else 'false'}", "trainer.resume_mode=none"])


def batch(seed, B=6, P=40, R=24, vocab=2048):
    g = torch.Generator().manual_seed(seed)
    seq = torch.randint(4, vocab, (B, P + R), generator=g)
    att = torch.ones(B, P + R, dtype=torch.long)
    rmask = torch.ones(B, R)
    adv = torch.randn(B, R, generator=g) / (B * R)
    old = -torch.rand(B, R, generator=g)
    b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                            "advantages": adv, "action_log_probs": old, "rollout_logprobs": None,
                            "base_action_log_probs": None})
    b.metadata = {"uids": [f"u{i // 2}" for i in range(B)]}
    return b


def main():
    env = pdist.init_distributed()
    assert env.world_size == 2 and env.device.type == "cuda"
    ctx = PeerContext(env.device)
    results = []
    for overlap in (False, True):
        w = PolicyWorker(cfg(overlap).trainer, model_path="tiny-qwen2-d128", env=env, peer_ctx=ctx, seed=0)
        assert w.optimizer.transport == "peer"
        norms = []
        for step in range(3):
            w.forward_backward(batch(100 * step + env.rank), step_follows=True)  # three micro-batches of two rows
            if overlap:
                assert len(w.optimizer._buckets_done) == w.model.args.num_layers, w.optimizer._buckets_done
            norms.append(float(w.optim_step()))
            assert not w.optimizer._buckets_done
        torch.cuda.synchronize()
        results.append((w.model.flat_params.clone(), norms))
        assert _lib.status_read_clear() == 0
    (p0, n0), (p1, n1) = results
    assert torch.equal(p0, p1), (p0.float() - p1.float()).abs().max()
    assert all(abs(a - b) <= 1e-5 * max(1.0, abs(a)) for a, b in zip(n0, n1)), (n0, n1)
    assert all(x > 0 for x in n0)
    dist.barrier()
    if env.rank == 0:
        print("OVERLAP_REDUCE_OK", n1)
    pdist.shutdown()


if __name__ == "__main__":
    main()
