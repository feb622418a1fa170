"""Run under torchrun, world size 2 (gloo on CPU, NCCL + peer memory on GPUs): a tensor-parallel engine must emit the
same greedy tokens and log-probabilities as the unsharded engine on the same weights and prompts."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from skyrl_b200.engine.llm_engine import EngineConfig, LLMEngine, SamplingParams  # noqa: E402
from skyrl_b200.engine.tp_model import TPEngineModel  # noqa: E402
from skyrl_b200.models.decoder import PRESETS, CausalLM  # noqa: E402
from skyrl_b200.ops import _lib  # noqa: E402
from skyrl_b200.parallel import dist as pdist  # noqa: E402
from skyrl_b200.parallel import tensor_parallel as tpm  # noqa: E402


def main():
    cuda = torch.cuda.is_available() and os.environ.get("SB_FORCE_CPU", "0") != "1"
    env = pdist.init_distributed(device=None if cuda else "cpu", backend=None if cuda else "gloo")
    dev = env.device
    dtype = torch.bfloat16 if cuda else torch.float32
    name = sys.argv[1] if len(sys.argv) > 1 else ("tiny-qwen2-tp" if cuda else "tiny-llama")
    a = PRESETS[name]
    full = CausalLM(a, device=dev, dtype=dtype, seed=3)
    peer = None
    if cuda:
        from skyrl_b200.parallel.peer import PeerContext

        peer = PeerContext(dev)
    tp = tpm.TPGroup(peer, None)
    assert tp.size == 2
    tpm_model = TPEngineModel(a, tp, device=dev, dtype=dtype)
    tpm_model.load_from_full(full)
    g = torch.Generator().manual_seed(11)
    lens = [17, 40, 9, 33, 64, 5]
    prompts = [torch.randint(4, a.vocab_size, (L,), generator=g).tolist() for L in lens]
    new = [12, 20, 7, 16, 9, 24]
    sps = [SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True) for n in new]

    def run(model, eager):
        eng = LLMEngine(model, EngineConfig(block_size=16, num_blocks=256, max_num_seqs=8, max_model_len=128,
                                            max_num_batched_tokens=256, enforce_eager=eager, sync_interval=4, seed=5))
        return eng.generate(prompts, sps)

    ref = run(full, True)
    modes = [True, False] if cuda else [True]
    for eager in modes:
        got = run(tpm_model, eager)
        for r, o in zip(ref, got):
            assert len(o.token_ids) == len(r.token_ids)
            lp_err = max(abs(x - y) for x, y in zip(o.logprobs, r.logprobs))
            if cuda:
                # bf16: partial sums are rounded in a different order than in the unsharded GEMM, so a near-tie can
                # flip late in a sequence; the first tokens and the log-probs of agreeing prefixes must match
                agree = 0
                for x, y in zip(o.token_ids, r.token_ids):
                    if x != y:
                        break
                    agree += 1
                assert agree >= min(4, len(r.token_ids)), (agree, o.token_ids[:8], r.token_ids[:8])
                pre = max(abs(x - y) for x, y in zip(o.logprobs[:agree], r.logprobs[:agree]))
                assert pre < 0.08, pre
            else:
                assert o.token_ids == r.token_ids, (o.token_ids, r.token_ids)
                assert lp_err < 1e-4, lp_err
        # both ranks produced identical outputs without exchanging a token
        mine = [(o.token_ids, [round(x, 6) for x in o.logprobs]) for o in got]
        parts = [None, None]
        dist.all_gather_object(parts, mine)
        assert parts[0] == parts[1], "the tensor-parallel ranks diverged"
    if cuda:
        torch.cuda.synchronize()
        assert _lib.status_read_clear() == 0
    dist.barrier()
    if env.rank == 0:
        print(f"ENGINE_TP_OK model={name} cuda={cuda}")
    pdist.shutdown()


if __name__ == "__main__":
    main()
