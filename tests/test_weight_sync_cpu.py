"""Weight-sync plumbing on CPU: chunk grouping / packing, strategy selection, delta publish -> fetch -> replay."""
import json
import os

import pytest
import torch

from skyrl_b200.models.decoder import CausalLM, ModelArgs
from skyrl_b200.models import hf_io
from skyrl_b200.weight_sync import (BroadcastStrategy, FlatModelWeightExtractor, WeightChunk, load_chunk_into_model,
                                    select_strategy_name)
from skyrl_b200.weight_sync.delta import DeltaPublisher, LocalCheckpointStore
from skyrl_b200.weight_sync.extractor import module_of


def _model(seed=0):
    args = ModelArgs(vocab_size=64, hidden_size=32, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=16,
                     intermediate_size=48, attention_bias=True, tie_word_embeddings=False)
    return CausalLM(args, dtype=torch.bfloat16, seed=seed)


def test_chunks_group_qkv_together_and_respect_threshold():
    m = _model()
    ex = FlatModelWeightExtractor(m, threshold_gb=4096 / (1 << 30))
    chunks = list(ex.extract_weights(torch.bfloat16))
    assert sum(len(c) for c in chunks) == len(hf_io.to_hf_state_dict(m))
    for c in chunks:
        mods = {}
        for n in c.names:
            mods.setdefault(module_of(n), []).append(n)
        for mod, names in mods.items():
            if mod.endswith("self_attn"):  # q, k, v (+ biases) and o arrive together for fused loaders
                assert {"q_proj", "k_proj", "v_proj"} <= {n.split(".")[-2] for n in names}
    assert module_of("model.layers.0.self_attn.q_proj.weight") == "model.layers.0.self_attn"
    c = chunks[0]
    rt = WeightChunk.unpack(c.names, c.dtypes, c.shapes, c.pack())
    assert all(torch.equal(a, b) for a, b in zip(rt.tensors, c.tensors))
    with pytest.raises(ValueError):
        WeightChunk(["a"], [], [], [])


def test_broadcast_strategy_single_process_loads_into_other_model():
    src, dst = _model(1), _model(2)
    assert not torch.equal(src.flat_params, dst.flat_params)
    st = BroadcastStrategy(on_chunk=lambda req, packed: load_chunk_into_model(dst, req, packed))
    moved = st.send(FlatModelWeightExtractor(src).extract_weights(torch.bfloat16))
    assert moved == sum(v.numel() * 2 for v in hf_io.to_hf_state_dict(src).values())
    for k, v in hf_io.to_hf_state_dict(src).items():
        assert torch.equal(v, hf_io.to_hf_state_dict(dst)[k]), k


def test_strategy_selection():
    assert select_strategy_name("nccl", True, True) == "in_place"
    assert select_strategy_name("nccl", False, True) == "peer"
    assert select_strategy_name("nccl", False, False) == "broadcast"
    assert select_strategy_name("nccl", False, True, delta_cfg=object()) == "delta"


def test_delta_publish_fetch_replay_and_recovery(tmp_path):
    m = _model(3)
    sync, local = str(tmp_path / "sync"), str(tmp_path / "local")
    pub = DeltaPublisher(sync, max_file_bytes=2048)
    pub.publish_base(hf_io.to_hf_state_dict(m))
    versions = {0: {k: v.clone() for k, v in hf_io.to_hf_state_dict(m).items()}}
    for v in (1, 2, 3):
        with torch.no_grad():
            m.p("layers.0.wo").add_(0.01 * v)
            m.p("final_norm").mul_(1.0 + 0.001 * v)
        d = pub.publish(hf_io.to_hf_state_dict(m))
        man = json.load(open(os.path.join(d, "manifest.json")))
        changed = {e["name"] for e in man["tensors"] if e["changed"]}
        assert "model.layers.0.self_attn.o_proj.weight" in changed and "model.embed_tokens.weight" not in changed
        versions[v] = {k: t.clone() for k, t in hf_io.to_hf_state_dict(m).items()}
    store = LocalCheckpointStore(sync, local)
    assert store.fetch(2) == 2
    for k, t in store.state_dict().items():
        assert torch.equal(t, versions[2][k]), k
    # a second store instance resumes from the persisted copy and only replays delta 3
    store2 = LocalCheckpointStore(sync, local)
    assert store2.fetch(3) == 3
    assert all(torch.equal(t, versions[3][k]) for k, t in store2.state_dict().items())
    # crash in the middle of a write: the marker forces a rebuild from the base
    store2._write_state(3, True)
    store3 = LocalCheckpointStore(sync, local)
    assert store3.fetch(3) == 3 and all(torch.equal(t, versions[3][k]) for k, t in store3.state_dict().items())
    # corrupted payload is detected by the checksum
    d1 = os.path.join(sync, "delta-00000001")
    payload = [f for f in os.listdir(d1) if f.startswith("payload")][0]
    raw = bytearray(open(os.path.join(d1, payload), "rb").read())
    raw[len(raw) // 2] ^= 0xFF
    open(os.path.join(d1, payload), "wb").write(bytes(raw))
    fresh = LocalCheckpointStore(sync, str(tmp_path / "local2"))
    with pytest.raises(Exception):
        fresh.fetch(1)


def test_delta_publish_of_unchanged_weights_still_advances_the_version(tmp_path):
    m = _model(3)
    sync = str(tmp_path / "sync")
    pub = DeltaPublisher(sync)
    pub.publish_base(hf_io.to_hf_state_dict(m))
    d = pub.publish(hf_io.to_hf_state_dict(m))
    man = json.load(open(os.path.join(d, "manifest.json")))
    assert d.endswith("delta-00000001") and not any(e["changed"] for e in man["tensors"])
    store = LocalCheckpointStore(sync, str(tmp_path / "local"))
    assert store.fetch(1) == 1
    want = hf_io.to_hf_state_dict(m)
    assert all(torch.equal(t, want[k]) for k, t in store.state_dict().items())
    # a late joiner replays every version it missed
    with torch.no_grad():
        m.p("final_norm").mul_(1.5)
    pub.publish(hf_io.to_hf_state_dict(m))
    with torch.no_grad():
        m.p("layers.0.wo").add_(0.25)
    pub.publish(hf_io.to_hf_state_dict(m))
    late = LocalCheckpointStore(sync, str(tmp_path / "late"))
    assert late.fetch(3) == 3
    want = hf_io.to_hf_state_dict(m)
    assert all(torch.equal(t, want[k]) for k, t in late.state_dict().items())
