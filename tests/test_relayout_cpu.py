"""Weight-sync re-layout plan: shards of a tensor-parallel trainer reach engine shards of another tensor-parallel
degree bit-exactly, compared with gather-then-slice (the reference's dataflow)."""
import dataclasses

import pytest
import torch

from skyrl_b200.models.decoder import PRESETS, CausalLM
from skyrl_b200.models.tp_decoder import local_args, shard_param
from skyrl_b200.weight_sync import relayout as rl


def _shard_model(full: CausalLM, tp: int, r: int) -> CausalLM:
    m = CausalLM(local_args(full.args, tp) if tp > 1 else full.args, device="cpu", dtype=full.flat_params.dtype, seed=None)
    with torch.no_grad():
        for name, prm in m.named_flat_views():
            prm.copy_(shard_param(name, full.p(name).detach(), full.args, tp, r) if tp > 1 else full.p(name))
    return m


@pytest.mark.parametrize("src_tp,dst_tp", [(4, 2), (2, 1), (1, 2), (2, 2), (4, 1), (2, 4)])
@pytest.mark.parametrize("model", ["tiny-qwen2-tp", "tiny-llama"])
def test_plan_reaches_every_engine_shard_bit_exactly(src_tp, dst_tp, model):
    a = PRESETS[model]
    if a.num_kv_heads % max(src_tp, dst_tp) or a.num_heads % max(src_tp, dst_tp):
        a = dataclasses.replace(a, num_heads=8, num_kv_heads=4)
    full = CausalLM(a, device="cpu", dtype=torch.float32, seed=1)
    srcs = [_shard_model(full, src_tp, r) for r in range(src_tp)]
    want = [_shard_model(full, dst_tp, e) for e in range(dst_tp)]
    # destinations: one engine shard per GPU of the source group (engine replicas repeat when dst_tp < src_tp)
    n_gpu = max(src_tp, dst_tp)
    got = [CausalLM(want[g % dst_tp].args, device="cpu", dtype=torch.float32, seed=None) for g in range(n_gpu)]
    for g in got:
        g.flat_params.fill_(float("nan"))
    dests = [rl.Destination(0, got[g].offsets, dst_tp, g % dst_tp, tensor=got[g].flat_params) for g in range(n_gpu)]
    total = 0
    for r in range(src_tp):
        plan = rl.build_plan(a, srcs[r].offsets, src_tp, r, dests)
        rl.run_plan_reference(plan, srcs[r].flat_params, dests)
        total += sum(c.rows * c.cols for c in plan)
    for g in range(n_gpu):
        for name, prm in got[g].named_flat_views():
            assert torch.equal(prm, want[g % dst_tp].p(name)), (name, g)
    # nothing is sent twice: the elements moved equal the elements the destinations hold
    assert total == sum(sum(n for _, n in d.offsets.values()) for d in dests)


def test_plan_blocks_are_vector_aligned_for_the_benchmark_models():
    for model, src_tp, dst_tp in (("qwen2.5-7b", 4, 2), ("qwen2.5-1.5b", 2, 1), ("qwen2.5-7b", 2, 2)):
        a = PRESETS[model]
        src = CausalLM.__new__(CausalLM)
        from skyrl_b200.models.decoder import _align, _param_specs
        import math

        def offsets(args):
            off, out = 0, {}
            for name, shape in _param_specs(args):
                out[name] = (off, math.prod(shape))
                off += _align(math.prod(shape))
            return out

        so = offsets(local_args(a, src_tp))
        do = offsets(local_args(a, dst_tp) if dst_tp > 1 else a)
        for r in range(src_tp):
            dests = [rl.Destination(0, do, dst_tp, g % dst_tp) for g in range(src_tp)]
            for c in rl.build_plan(a, so, src_tp, r, dests):
                assert c.cols % 8 == 0 and c.src_off % 8 == 0 and c.dst_off % 8 == 0, c
                assert c.rows == 1 or (c.src_ld % 8 == 0 and c.dst_ld % 8 == 0), c


@pytest.mark.parametrize("src_tp,replicas", [(1, 4), (2, 2), (1, 3)])
def test_data_parallel_replicas_share_the_push(src_tp, replicas):
    """Disaggregated engines fed by a data-parallel trainer: every replica pushes a disjoint part, together everything."""
    a = PRESETS["tiny-qwen2-tp"]
    full = CausalLM(a, device="cpu", dtype=torch.float32, seed=2)
    srcs = [_shard_model(full, src_tp, r) for r in range(src_tp)]
    got = [CausalLM(a, device="cpu", dtype=torch.float32, seed=None) for _ in range(2)]  # two unsharded remote engines
    for g in got:
        g.flat_params.fill_(float("nan"))
    dests = [rl.Destination(0, g.offsets, 1, 0, tensor=g.flat_params) for g in got]
    total = 0
    for r in range(src_tp):
        for k in range(replicas):
            plan = rl.build_plan(a, srcs[r].offsets, src_tp, r, dests, chunk_world=replicas, chunk_rank=k)
            rl.run_plan_reference(plan, srcs[r].flat_params, dests)
            total += sum(c.rows * c.cols for c in plan)
    for g in got:
        for name, prm in g.named_flat_views():
            assert torch.equal(prm, full.p(name)), name
    assert total == 2 * sum(n for _, n in got[0].offsets.values())
