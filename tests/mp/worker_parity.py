"""Run under torchrun on CPU (gloo), world size 2:  python worker_parity.py {tp|sp|ep|pp}

Worker-level parity of the model-parallel strategies: after one ``forward_backward`` + ``optim_step`` through the
``PolicyWorker`` (the code path the trainer drives), the full parameters must equal those of a single-rank worker that
trained on the same data, replicas inside a model-parallel group must be identical, and the trainer's mini-batch
arithmetic must give one optimizer step per RL step when ``train_batch_size == policy_mini_batch_size``.
"""
import os
import sys
from types import SimpleNamespace

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.config.config import SkyRLTrainConfig  # noqa: E402
from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.parallel.sharded_optimizer import ShardedAdamW  # noqa: E402
from skyrl_b200.train.batch import TrainingInputBatch  # noqa: E402
from skyrl_b200.workers.worker import PolicyWorker  # noqa: E402

MODELS = {"tp": "tiny-llama", "sp": "tiny-llama", "pp": "tiny-llama", "pp_mb1": "tiny-llama", "ep": "tiny-moe", "tpv": "tiny-llama",
          "critic_tp": "tiny-llama", "critic_sp": "tiny-llama", "cp": "tiny-llama", "cp_megatron": "tiny-llama",
          "critic_cp": "tiny-llama"}


def cfg_for(mode: str, model: str):
    extra = {
        "tp": ["trainer.strategy=megatron", "trainer.policy.megatron_config.tensor_model_parallel_size=2"],
        "sp": ["trainer.policy.sequence_parallel_size=2"],
        "ep": ["trainer.strategy=megatron", "trainer.policy.megatron_config.expert_model_parallel_size=2"],
        "pp": ["trainer.strategy=megatron", "trainer.policy.megatron_config.pipeline_model_parallel_size=2"],
        # four micro-batches in flight through the two stages
        "pp_mb1": ["trainer.strategy=megatron", "trainer.policy.megatron_config.pipeline_model_parallel_size=2",
                   "trainer.micro_train_batch_size_per_gpu=1", "trainer.gradient_checkpointing=true"],
        "tpv": ["trainer.strategy=megatron", "trainer.policy.megatron_config.tensor_model_parallel_size=2",
                "trainer.b200.vocab_parallel_lm_head=true"],
        "critic_tp": ["trainer.strategy=megatron", "trainer.policy.megatron_config.tensor_model_parallel_size=2"],
        "critic_sp": ["trainer.critic.sequence_parallel_size=2", "trainer.policy.sequence_parallel_size=2"],
        "cp": ["trainer.policy.sequence_parallel_size=2", "trainer.sequence_parallel_backend=context"],
        "cp_megatron": ["trainer.strategy=megatron", "trainer.policy.megatron_config.context_parallel_size=2"],
        "critic_cp": ["trainer.critic.sequence_parallel_size=2", "trainer.policy.sequence_parallel_size=2",
                      "trainer.sequence_parallel_backend=context"],
        "none": [],
    }[mode]
    return SkyRLTrainConfig.from_cli_overrides([
        f"trainer.policy.model.path={model}", "trainer.train_batch_size=4", "trainer.policy_mini_batch_size=4",
        "trainer.micro_train_batch_size_per_gpu=2", "generator.n_samples_per_prompt=2", "trainer.bf16=false",
        "trainer.algorithm.use_kl_loss=false", "trainer.policy.optimizer_config.lr=1e-3",
        "trainer.policy.optimizer_config.max_grad_norm=0.5", "trainer.gradient_checkpointing=false",
        "trainer.critic.optimizer_config.lr=1e-3", "trainer.critic.optimizer_config.max_grad_norm=0.5",
        "trainer.max_tokens_per_microbatch=0", "trainer.resume_mode=none", *extra])


def make_batch(seed: int, B: int = 4, P: int = 12, R: int = 10, vocab: int = 1024) -> TrainingInputBatch:
    g = torch.Generator().manual_seed(seed)
    seq = torch.randint(4, vocab, (B, P + R), generator=g)
    att = torch.ones(B, P + R, dtype=torch.long)
    att[1, :3] = 0  # left padding
    rmask = torch.ones(B, R)
    rmask[2, -4:] = 0
    att[2, -4:] = 0
    adv = torch.randn(B, R, generator=g) * rmask / rmask.sum()
    old = -torch.rand(B, R, generator=g)
    b = TrainingInputBatch({"sequences": seq, "attention_mask": att, "response_mask": rmask, "loss_mask": rmask.clone(),
                            "advantages": adv, "action_log_probs": old, "rollout_logprobs": None,
                            "base_action_log_probs": None, "values": torch.randn(B, R, generator=g) * 0.1,
                            "returns": torch.randn(B, R, generator=g)})
    b.metadata = {"uids": [f"u{i // 2}" for i in range(B)]}
    return b


def full_state(worker) -> dict:
    """Name -> full (unsharded) parameter, identical on every rank."""
    m = worker.model
    if hasattr(m, "gather_full_state"):
        return {k: v.detach().float().clone() for k, v in m.gather_full_state().items()}
    if worker.pipe is not None:  # each stage owns a layer range: exchange the named views
        mine = {k: v.detach().float().clone() for k, v in m.named_flat_views()}
        parts = [None] * dist.get_world_size()
        dist.all_gather_object(parts, mine)
        out = {}
        for p in parts:
            out.update({k: v for k, v in p.items() if k not in out})
        return out
    return {k: v.detach().float().clone() for k, v in m.named_flat_views()}


def main():
    mode = sys.argv[1]
    env = pdist.init_distributed(backend="gloo", device="cpu")
    assert env.world_size == 2
    model = MODELS[mode]
    solo = [dist.new_group([r]) for r in range(2)][env.rank]

    # ---- model-parallel worker
    from skyrl_b200.workers.worker import CriticWorker

    Worker = CriticWorker if mode.startswith("critic") else PolicyWorker
    w = Worker(cfg_for(mode, model).trainer, model_path=model, env=env, seed=0)
    if mode in ("cp", "cp_megatron", "critic_cp"):
        assert type(w.model).__name__ == "ContextParallelCausalLM"
    if mode == "tpv":
        assert w.model.vocab_parallel_head and w.model.p("lm_head").shape[0] == 512
    if mode == "ep":
        batches = [make_batch(100), make_batch(101)]  # expert-parallel ranks keep their own data
        local = batches[env.rank]
    else:
        batches = [make_batch(100)]
        local = batches[0]
    st = w.forward_backward(local)
    gn = float(w.optim_step())
    got = full_state(w)

    # ---- single-rank reference on the same data (both ranks compute it redundantly)
    one = pdist.DistEnv(0, 0, 1, torch.device("cpu"))
    ref = Worker(cfg_for("none", model).trainer, model_path=model, env=one, seed=0)
    o = ref.optimizer
    ref.optimizer = ShardedAdamW(ref.model.flat_params, ref.flat_grad, lr=o.lr, betas=o.betas, weight_decay=o.weight_decay,
                                 max_grad_norm=o.max_grad_norm, group=solo)
    from skyrl_b200.parallel.sharded_optimizer import get_scheduler

    oc = getattr(cfg_for("none", model).trainer, "critic" if mode.startswith("critic") else "policy").optimizer_config
    ref.scheduler = get_scheduler(oc.scheduler, ref.optimizer, oc.num_warmup_steps, base_lr=oc.lr)
    for b in batches:
        if mode == "ep":  # two data shards: each contributes half of the KL / entropy weights, advantages are pre-scaled
            b = b
        ref.forward_backward(b)
    gn_ref = float(ref.optim_step())
    want = {k: v.detach().float() for k, v in ref.model.named_flat_views()}

    # ---- checks
    assert abs(gn - gn_ref) <= 2e-4 * max(1.0, abs(gn_ref)), (mode, gn, gn_ref)
    worst = 0.0
    for k, v in want.items():
        assert k in got, f"{k} missing from the gathered state"
        err = (got[k] - v).abs().max().item()
        worst = max(worst, err)
        assert err < 2e-5, (mode, k, err)
    moved = max((want[k] - dict(Worker(cfg_for("none", model).trainer, model_path=model, env=one, seed=0)
                                .model.named_flat_views())[k].float()).abs().max().item() for k in list(want)[:3])
    assert moved > 1e-4, "the reference update did not move the parameters"
    # replicas inside the group are bit-identical
    for k, v in got.items():
        other = [torch.empty_like(v) for _ in range(2)]
        dist.all_gather(other, v.contiguous())
        assert torch.equal(other[0], other[1]), (mode, k)

    # ---- trainer arithmetic: one optimizer step per RL step, advantages scaled by the number of data shards
    from skyrl_b200.train.trainer import PPOTrainer

    tr = PPOTrainer.__new__(PPOTrainer)
    tr.cfg, tr.env = cfg_for(mode, model), env
    calls = {"fb": 0, "opt": 0, "rows": []}

    def fb(mini, **kw):
        calls["fb"] += 1
        calls["rows"].append(mini.batch_size)
        return {}

    def opt():
        calls["opt"] += 1
        return None

    if mode.startswith("critic"):
        dist.barrier()
        if env.rank == 0:
            print(f"WORKER_PARITY_OK mode={mode} grad_norm={gn:.6f} max_param_err={worst:.2e}")
        pdist.shutdown()
        return
    share = 1 if mode == "ep" else 2
    tr.policy = SimpleNamespace(tp_size=share, forward_backward=fb, optim_step=opt)
    tr.critic = None
    nb = 4 * 2 * share // 2  # rows held by this rank: train_batch * n_samples / dp
    merged = make_batch(7, B=nb)
    merged.metadata = {"uids": [f"u{i // 2}" for i in range(nb)]}
    tr._execute_training_step("policy", merged)
    assert calls["opt"] == 1 and calls["fb"] == 1 and calls["rows"] == [nb], calls
    raw = make_batch(8, B=nb)
    raw["advantages"] = torch.ones_like(raw["advantages"])
    mk = raw["loss_mask"]
    out = tr._normalize_advantages(raw)
    dp = 2 // share
    want_scale = 1.0 / (float(mk.sum()) * dp)  # every data shard holds the same mask here
    assert abs(float(out["advantages"][0, 0]) - want_scale) < 1e-7 * max(1.0, want_scale), (float(out["advantages"][0, 0]), want_scale)
    dist.barrier()
    if env.rank == 0:
        print(f"WORKER_PARITY_OK mode={mode} grad_norm={gn:.6f} max_param_err={worst:.2e}")
    pdist.shutdown()


if __name__ == "__main__":
    main()
