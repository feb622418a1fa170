"""Run under torchrun on 2 GPUs: the weight-sync re-layout kernel (peer stores from the owning trainer shard into the
engines' buffers) is bit-exact against gather-then-slice, for an unsharded and for a tensor-parallel engine."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.config.config import SkyRLTrainConfig  # noqa: E402
from skyrl_b200.models.tp_decoder import shard_param  # noqa: E402
from skyrl_b200.ops import _lib  # noqa: E402
from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.workers.worker import PolicyWorker  # noqa: E402


def cfg(tp):
    extra = ["trainer.strategy=megatron", f"trainer.policy.megatron_config.tensor_model_parallel_size={tp}"] if tp > 1 else []
    return SkyRLTrainConfig.from_cli_overrides(["trainer.policy.model.path=tiny-qwen2-tp", "trainer.resume_mode=none", *extra])


def main():
    env = pdist.init_distributed()
    assert env.world_size == 2 and env.device.type == "cuda"
    for trainer_tp, engine_tp in ((2, 1), (2, 2), (1, 2)):
        w = PolicyWorker(cfg(trainer_tp).trainer, model_path="tiny-qwen2-tp", env=env, seed=trainer_tp * 10 + engine_tp)
        with torch.no_grad():  # distinct values everywhere, so a misplaced block cannot go unnoticed
            w.model.flat_params.copy_(torch.randn(w.model.flat_params.numel(), device=env.device) * 0.05)
            if trainer_tp > 1:
                w.model.reduce_replicated_grads()  # no-op for values; replicated leaves are made equal below
                for name, prm in w.model.named_flat_views():
                    if name.split(".")[-1] in ("embed", "ln1", "ln2", "final_norm", "lm_head"):
                        dist.broadcast(prm.data, src=0)
            else:
                dist.broadcast(w.model.flat_params, src=0)
        ec = w.engine_model(engine_tp)
        assert w._relayout is not None and w._relayout.n_desc > 0
        for _ in range(2):  # a second sync after a weight change
            with torch.no_grad():
                w.model.flat_params.mul_(1.5)
            w.refresh_engine_model()
            torch.cuda.synchronize()
            full = w.model.gather_full_state() if trainer_tp > 1 else dict(w.model.named_flat_views())
            fa = w.model.full_args if trainer_tp > 1 else w.model.args
            for name, prm in ec.named_flat_views():
                want = shard_param(name, full[name], fa, engine_tp, env.rank % engine_tp) if engine_tp > 1 else full[name]
                assert torch.equal(prm, want), (trainer_tp, engine_tp, name)
            dist.barrier()  # a peer's next push must not land while this rank still compares (in training the step
            # structure provides this ordering: engines are idle while weights are pushed)
        assert w.last_weight_sync_ms > 0 and _lib.status_read_clear() == 0
        if env.rank == 0:
            print(f"relayout trainer_tp={trainer_tp} engine_tp={engine_tp}: {w._relayout.n_desc} block copies, "
                  f"{w.last_weight_sync_bytes / 1e6:.2f} MB out, {w.last_weight_sync_ms:.3f} ms")
    dist.barrier()
    if env.rank == 0:
        print("RELAYOUT_OK")
    pdist.shutdown()


if __name__ == "__main__":
    main()
