"""Pin the models to HF transformers, the oracle the reference validated its engine against
(reports/11_custom_engine.md:25-38: prefill logits, fixed-trajectory decode logits, argmax agreement
over 24 steps).  A tiny random ``LlamaForCausalLM`` is built, saved in the HF safetensors layout and
loaded back through ``SafetensorsSource`` + ``shard_for_rank``:

  * CPU, fp32: this repository's plain-PyTorch model (the oracle of the kernel tests) must reproduce
    HF's logits to float rounding, prefill and every decode step on HF's own greedy trajectory;
  * GPU, bf16: the engine (sm_100a kernels, paged cache, captured decode step) must agree with HF run
    in bf16 on the same device within bf16 tolerance, and pick the same token wherever HF's top-2
    margin is larger than that tolerance.
Skipped where transformers is not importable."""
import pytest
import torch

transformers = pytest.importorskip("transformers")
STEPS = 24


def _tiny_hf(tmp_path, dtype, seed=11):
    from libtbvcoll_b200.models.config import get_config
    cfg = get_config("tiny")
    hc = transformers.LlamaConfig(
        hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_layers,
        num_attention_heads=cfg.num_heads, num_key_value_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, vocab_size=cfg.vocab_size,
        rms_norm_eps=cfg.rms_eps, rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_position, tie_word_embeddings=False,
        attention_bias=False, mlp_bias=False, hidden_act="silu")
    torch.manual_seed(seed)
    model = transformers.LlamaForCausalLM(hc).to(dtype).eval()
    with torch.no_grad():                       # norms away from 1 and larger weights: a layout mistake must show
        for n, p in model.named_parameters():
            if n.endswith("norm.weight"):
                p.copy_(1.0 + 0.1 * torch.randn_like(p))
            else:
                p.mul_(2.0)
    model.save_pretrained(str(tmp_path), safe_serialization=True)
    return cfg, model


def _hf_trajectory(model, prompt, device):
    """HF greedy continuation and the logits HF assigns at every position of prompt + continuation."""
    ids = torch.tensor([prompt], device=device)
    with torch.no_grad():
        seq = model.generate(ids, max_new_tokens=STEPS, do_sample=False, use_cache=True, pad_token_id=0)
        logits = model(seq).logits[0].float()
    return seq[0].tolist(), logits


def test_plain_pytorch_model_reproduces_hf_transformers_fp32(tmp_path):
    from libtbvcoll_b200.models.config import from_hf_config
    from libtbvcoll_b200.models.torch_baseline import TorchLlamaTP
    from libtbvcoll_b200.utils.weights import SafetensorsSource, shard_for_rank
    cfg, hf = _tiny_hf(tmp_path, torch.float32)
    loaded = from_hf_config(str(tmp_path / "config.json"))
    assert (loaded.hidden_size, loaded.num_layers, loaded.num_heads, loaded.num_kv_heads, loaded.intermediate_size, loaded.vocab_size) == \
           (cfg.hidden_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.intermediate_size, cfg.vocab_size)
    w = shard_for_rank(cfg, SafetensorsSource(str(tmp_path), dtype=torch.float32), 0, 1, "cpu", interleave_gate_up=False)
    ours = TorchLlamaTP(cfg, 0, 1, w, "cpu", max_batch=1, max_seq_len=128)
    prompt = torch.randint(0, cfg.vocab_size, (19,), generator=torch.Generator().manual_seed(2)).tolist()
    seq, want = _hf_trajectory(hf, prompt, "cpu")
    L = len(prompt)
    with torch.no_grad():
        got = ours.forward(torch.tensor([prompt]), torch.arange(L, dtype=torch.int32)[None], 0)[0]
        scale = want.abs().max().item()
        assert (got - want[L - 1]).abs().max().item() <= 2e-4 * scale                  # prefill logits
        agree = int(got.argmax() == want[L - 1].argmax())
        for t in range(STEPS - 1):                                                     # HF's trajectory, one token at a time
            pos = L + t
            got = ours.forward(torch.tensor([[seq[pos]]]), torch.tensor([[pos]], dtype=torch.int32), pos)[0]
            assert (got - want[pos]).abs().max().item() <= 2e-4 * scale, t
            agree += int(got.argmax() == want[pos].argmax())
    assert agree == STEPS


@pytest.mark.gpu
def test_engine_agrees_with_hf_transformers_bf16(tmp_path):
    from libtbvcoll_b200.engine.engine import Engine
    from libtbvcoll_b200.utils.weights import SafetensorsSource
    dev = "cuda:0"
    cfg, hf = _tiny_hf(tmp_path, torch.bfloat16)
    hf = hf.to(dev)
    eng = Engine(cfg, device=dev, source=SafetensorsSource(str(tmp_path)), max_batch=1, max_seq_len=128, prefill_chunk=64)
    prompt = torch.randint(0, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(3)).tolist()
    seq, want = _hf_trajectory(hf, prompt, dev)
    L = len(prompt)
    scale = want.abs().max().item()
    tol = 0.03 * scale + 0.02                        # bf16 activations through 2 layers, different summation orders

    def margin(row):
        top = row.topk(2).values
        return (top[0] - top[1]).item()

    eng.prefill([prompt], STEPS + 1)
    got = eng.model.logits[0].float().clone()
    errs = [(got - want[L - 1]).abs().max().item()]
    agree, decided = int(got.argmax() == want[L - 1].argmax()), int(margin(want[L - 1]) > 2 * tol)
    clear_disagree = int(margin(want[L - 1]) > 2 * tol and got.argmax() != want[L - 1].argmax())
    splits = eng.attn_splits_for(1, L + STEPS)
    for t in range(STEPS - 1):                       # fixed trajectory: feed HF's token, compare the logits
        pos = L + t
        eng._load_decode_inputs(1, [seq[pos]], [pos])
        eng._decode_step(1, splits, False)
        torch.cuda.synchronize()
        got = eng.model.logits[0].float().clone()
        errs.append((got - want[pos]).abs().max().item())
        same = bool(got.argmax() == want[pos].argmax())
        agree += int(same)
        clear = margin(want[pos]) > 2 * tol
        decided += int(clear)
        clear_disagree += int(clear and not same)
    assert max(errs) <= tol, (max(errs), tol)
    assert clear_disagree == 0                       # wherever HF's choice is not a near-tie, the engine makes it too
    assert agree >= STEPS - 3, (agree, decided)      # near-ties between random-weight logits may flip
    # and the engine's own greedy generation follows HF's while the choices are clear
    out = eng.generate([prompt], STEPS)[0]
    first_diff = next((i for i, (a, b) in enumerate(zip(out, seq[L:])) if a != b), STEPS)
    assert first_diff >= 1
