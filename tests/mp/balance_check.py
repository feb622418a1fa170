"""Run under torchrun on CPU (gloo), world size 2 or 4:  python balance_check.py

Token balancing across data-parallel ranks: the plan equalises the loads, the exchange delivers every row exactly
once, and one policy update with balancing equals the update without it (the summed gradient is the same).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.config.config import SkyRLTrainConfig  # noqa: E402
from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.train.balance import balance_rows_across_ranks, plan_assignment  # noqa: E402
from skyrl_b200.train.batch import TrainingInputBatch  # noqa: E402
from skyrl_b200.train.trainer import PPOTrainer  # noqa: E402
from skyrl_b200.utils.tokenizer import SyntheticTokenizer  # noqa: E402


def make_batch(rank: int, B: int = 8, P: int = 6, R: int = 20) -> TrainingInputBatch:
    """Rank-dependent widths, like real rollouts: every rank pads to its own longest prompt and response."""
    P, R = P + rank, R - 2 * rank
    g = torch.Generator().manual_seed(100 + rank)
    # rank 0 holds long responses, the last rank short ones: a deliberately lopsided start
    hi = R if rank == 0 else max(3, R // (2 + rank))
    n_resp = torch.randint(2, hi + 1, (B,), generator=g)
    seq = torch.randint(4, 1024, (B, P + R), generator=g)
    att = torch.zeros(B, P + R, dtype=torch.long)
    rmask = torch.zeros(B, R)
    for i in range(B):
        lead = int(torch.randint(0, 3, (1,), generator=g))  # left padding of the prompt
        att[i, lead: P + int(n_resp[i])] = 1
        rmask[i, : int(n_resp[i])] = 1
    b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask.long(), "loss_mask": rmask.clone(),
                            "advantages": torch.randn(B, R, generator=g) * rmask, "action_log_probs": -torch.rand(B, R, generator=g),
                            "rollout_logprobs": None, "base_action_log_probs": None,
                            "row_tag": (torch.arange(B) + 1000 * rank).view(B, 1)})
    b.metadata = {"uids": [f"r{rank}u{i // 2}" for i in range(B)]}
    return b


def main():
    env = pdist.init_distributed(backend="gloo", device="cpu")
    W, rank = env.world_size, env.rank
    # ---- the plan alone
    lens = [[50, 40, 30, 20], [5, 5, 5, 5]]
    dest = plan_assignment(lens)
    load = [0, 0]
    cnt = [0, 0]
    for r in range(2):
        for i, d in enumerate(dest[r]):
            load[d] += lens[r][i]
            cnt[d] += 1
    assert cnt == [4, 4] and max(load) - min(load) <= 10, (dest, load)
    d2 = plan_assignment([[7, 7], [7, 7]])
    assert sorted(d2[0] + d2[1]) == [0, 0, 1, 1]  # two rows each, whatever their origin

    # ---- the exchange: every row arrives exactly once, fields stay aligned
    b = make_batch(rank)
    out, rep = balance_rows_across_ranks(b, rank, W)
    assert rep is not None and out.batch_size == b.batch_size
    assert rep["max_tokens_after"] <= rep["max_tokens_before"] and rep["max_tokens_after"] <= 1.1 * rep["mean_tokens"] + 26
    tags = [None] * W
    dist.all_gather_object(tags, out["row_tag"].view(-1).tolist())
    flat = sorted(t for ts in tags for t in ts)
    assert flat == sorted(i + 1000 * r for r in range(W) for i in range(b.batch_size)), "a row was lost or duplicated"
    src_rank = (out["row_tag"].view(-1) // 1000).tolist()
    src_row = (out["row_tag"].view(-1) % 1000).tolist()
    P_new = out["sequences"].shape[1] - out["response_mask"].shape[1]
    for j, (r, i) in enumerate(zip(src_rank, src_row)):
        ref = make_batch(r)
        P_r, R_r = ref["sequences"].shape[1] - ref["response_mask"].shape[1], ref["response_mask"].shape[1]
        # the row's real tokens, in order, and its response-aligned fields survive the move and the re-padding
        keep = out["attention_mask"][j].bool()
        assert out["sequences"][j][keep].tolist() == ref["sequences"][i][ref["attention_mask"][i].bool()].tolist(), j
        assert torch.equal(out["sequences"][j, P_new - P_r: P_new + R_r], ref["sequences"][i]), j
        for k in ("loss_mask", "advantages", "action_log_probs"):
            assert torch.equal(out[k][j, :R_r], ref[k][i]) and float(out[k][j, R_r:].abs().sum()) == 0.0, (k, j)
    assert out["rollout_logprobs"] is None and out.metadata["uids"] is None
    tot = torch.tensor([float(out["attention_mask"].sum())])
    allt = [torch.zeros(1) for _ in range(W)]
    dist.all_gather(allt, tot)
    assert max(float(t) for t in allt) == rep["max_tokens_after"]

    # ---- one policy update with and without balancing gives the same parameters
    def run(balance: bool):
        pdist_env = env
        cfg = SkyRLTrainConfig.from_cli_overrides([
            "trainer.policy.model.path=tiny-llama", f"trainer.train_batch_size={4 * W}", f"trainer.policy_mini_batch_size={4 * W}",
            "trainer.micro_train_batch_size_per_gpu=2", "generator.n_samples_per_prompt=2", "trainer.bf16=false",
            "trainer.algorithm.use_kl_loss=false", "trainer.policy.optimizer_config.lr=1e-3",
            "trainer.gradient_checkpointing=false", "trainer.max_tokens_per_microbatch=0", "trainer.resume_mode=none",
            f"trainer.b200.balance_tokens_across_ranks={'true' if balance else 'false'}"])
        tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024), env=pdist_env)
        from skyrl_b200.workers.worker import PolicyWorker

        tr.policy = PolicyWorker(cfg.trainer, model_path="tiny-llama", env=pdist_env, seed=0)
        tr.critic = None
        batch = make_batch(rank)
        del batch["row_tag"]
        m = tr._execute_training_step("policy", batch)
        return {k: v.detach().float().clone() for k, v in tr.policy.model.named_flat_views()}, m, dict(tr.all_metrics)

    p_off, m_off, _ = run(False)
    p_on, m_on, met = run(True)
    worst = max((p_on[k] - p_off[k]).abs().max().item() for k in p_off)
    assert worst < 2e-5, worst
    assert abs(m_on["grad_norm"] - m_off["grad_norm"]) < 1e-4 * max(1.0, m_off["grad_norm"])
    assert met["policy/token_imbalance_after"] <= met["policy/token_imbalance_before"]

    # ---- the summed gradient itself (an Adam step hides small gradient differences behind its normalisation)
    cfg = SkyRLTrainConfig.from_cli_overrides([
        "trainer.policy.model.path=tiny-llama", f"trainer.train_batch_size={4 * W}", f"trainer.policy_mini_batch_size={4 * W}",
        "trainer.micro_train_batch_size_per_gpu=2", "generator.n_samples_per_prompt=2", "trainer.bf16=false",
        "trainer.algorithm.use_kl_loss=true", "trainer.algorithm.kl_loss_coef=0.05", "trainer.gradient_checkpointing=false",
        "trainer.max_tokens_per_microbatch=0", "trainer.resume_mode=none"])
    from skyrl_b200.workers.worker import PolicyWorker

    tr = PPOTrainer(cfg, tokenizer=SyntheticTokenizer(1024), env=env)
    tr.policy = PolicyWorker(cfg.trainer, model_path="tiny-llama", env=env, seed=0)
    mini = make_batch(rank)
    del mini["row_tag"]
    mini["base_action_log_probs"] = mini["action_log_probs"] - 0.1  # a reference model, so the KL term takes part
    mini = tr._normalize_advantages(mini, None)
    grads = []
    for balanced in (False, True):
        mb = tr._balance_tokens(mini) if balanced else mini
        tr.policy.flat_grad.zero_()
        tr.policy.forward_backward(mb)
        g = tr.policy.flat_grad.detach().clone()
        dist.all_reduce(g)
        grads.append(g)
    tr.policy.flat_grad.zero_()
    rel_g = ((grads[0] - grads[1]).norm() / grads[0].norm()).item()
    assert grads[0].norm() > 0 and rel_g < 1e-5, rel_g
    dist.barrier()
    if rank == 0:
        print(f"BALANCE_OK world={W} imbalance {met['policy/token_imbalance_before']:.3f} -> "
              f"{met['policy/token_imbalance_after']:.3f} max_param_diff={worst:.2e} summed_grad_rel_diff={rel_g:.1e}")
    pdist.shutdown()


if __name__ == "__main__":
    main()
