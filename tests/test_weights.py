"""HF-layout weight sharding (no GPU): shards of every TP degree reassemble the same tensors."""
import torch

from libtbvcoll_b200.models.config import get_config, from_hf_config
from libtbvcoll_b200.utils.weights import RandomSource, SafetensorsSource, hf_tensor_shapes, save_hf_checkpoint, shard_for_rank


def test_shards_reassemble_full_tensors():
    cfg = get_config("tiny-bias")
    src = RandomSource(cfg, seed=1)
    full = shard_for_rank(cfg, src, 0, 1, "cpu", interleave_gate_up=False)
    for tp in (2, 4):
        shards = [shard_for_rank(cfg, src, r, tp, "cpu", interleave_gate_up=False) for r in range(tp)]
        assert torch.equal(torch.cat([s["embed"] for s in shards]), full["embed"])
        assert torch.equal(torch.cat([s["lm_head"] for s in shards]), full["lm_head"])
        d, nq, nkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
        for l in range(cfg.num_layers):
            q = torch.cat([s[f"layers.{l}.qkv.weight"][: nq // tp * d] for s in shards])
            assert torch.equal(q, full[f"layers.{l}.qkv.weight"][: nq * d])
            k = torch.cat([s[f"layers.{l}.qkv.weight"][nq // tp * d: (nq + nkv) // tp * d] for s in shards])
            assert torch.equal(k, full[f"layers.{l}.qkv.weight"][nq * d: (nq + nkv) * d])
            assert torch.equal(torch.cat([s[f"layers.{l}.o.weight"] for s in shards], 1), full[f"layers.{l}.o.weight"])
            assert torch.equal(torch.cat([s[f"layers.{l}.down.weight"] for s in shards], 1), full[f"layers.{l}.down.weight"])
            ipr = cfg.intermediate_size // tp
            gate = torch.cat([s[f"layers.{l}.gate_up.weight"][:ipr] for s in shards])
            assert torch.equal(gate, full[f"layers.{l}.gate_up.weight"][: cfg.intermediate_size])
            qb = torch.cat([s[f"layers.{l}.qkv.bias"][: nq // tp * d] for s in shards])
            assert torch.equal(qb, full[f"layers.{l}.qkv.bias"][: nq * d])


def test_kv_heads_replicate_when_tp_exceeds_them():
    cfg = get_config("tiny")            # 2 kv heads
    src = RandomSource(cfg, seed=2)
    d = cfg.head_dim
    s = [shard_for_rank(cfg, src, r, 4, "cpu") for r in range(4)]
    nq = cfg.num_heads // 4
    k = [x["layers.0.qkv.weight"][nq * d:(nq + 1) * d] for x in s]
    assert torch.equal(k[0], k[1]) and torch.equal(k[2], k[3]) and not torch.equal(k[0], k[2])


def test_interleaved_gate_up_layout():
    cfg = get_config("tiny")
    src = RandomSource(cfg, seed=3)
    a = shard_for_rank(cfg, src, 1, 2, "cpu", interleave_gate_up=True)["layers.1.gate_up.weight"]
    b = shard_for_rank(cfg, src, 1, 2, "cpu", interleave_gate_up=False)["layers.1.gate_up.weight"]
    ipr = cfg.intermediate_size // 2
    assert torch.equal(a[0::2], b[:ipr]) and torch.equal(a[1::2], b[ipr:])


def test_safetensors_round_trip_and_row_slices(tmp_path):
    cfg = get_config("tiny")
    src = RandomSource(cfg, seed=4)
    save_hf_checkpoint(src, str(tmp_path), max_shard_bytes=1 << 20)
    st = SafetensorsSource(str(tmp_path))
    assert set(st.names()) == set(hf_tensor_shapes(cfg))
    for n in list(st.names())[:6]:
        assert torch.equal(st.get(n), src.get(n))
    n = "model.layers.1.mlp.up_proj.weight"
    assert torch.equal(st.get_rows(n, 100, 228), src.get(n)[100:228])
    a = shard_for_rank(cfg, st, 1, 2, "cpu")
    b = shard_for_rank(cfg, src, 1, 2, "cpu")
    assert all(torch.equal(a[k], b[k]) for k in b)


def test_hf_config_json(tmp_path):
    import json
    p = tmp_path / "config.json"
    p.write_text(json.dumps({"model_type": "qwen2", "hidden_size": 3584, "num_hidden_layers": 28, "num_attention_heads": 28,
                             "num_key_value_heads": 4, "intermediate_size": 18944, "vocab_size": 152064, "rope_theta": 1e6,
                             "rms_norm_eps": 1e-6, "max_position_embeddings": 32768}))
    c = from_hf_config(str(p))
    assert c.head_dim == 128 and c.qkv_bias and c.num_kv_heads == 4 and c.param_count() > 7e9
