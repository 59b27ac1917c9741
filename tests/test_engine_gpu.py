"""The decode engine on one GPU: all decode loops agree bit for bit (the output-hash gate the
reference insists on for every performance change, reports/10_tp_custom_allreduce.md:420),
and the logits agree with the stock-PyTorch model within bf16 tolerance."""
import hashlib

import pytest
import torch

pytestmark = pytest.mark.gpu


def _hash(outs):
    return hashlib.sha256(repr(outs).encode()).hexdigest()


@pytest.mark.parametrize("name", ["tiny", "tiny-bias"])
def test_decode_loops_agree_and_match_torch_logits(name):
    from libtbvcoll_b200.engine.engine import Engine
    from libtbvcoll_b200.models.config import get_config
    from libtbvcoll_b200.models.torch_baseline import TorchLlamaTP
    from libtbvcoll_b200.utils.weights import RandomSource, shard_for_rank
    cfg = get_config(name)
    dev = "cuda:0"
    src = RandomSource(cfg, seed=3, device=dev)
    eng = Engine(cfg, device=dev, source=src, max_batch=4, max_seq_len=128, prefill_chunk=64)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (37, 5, 64, 20)]
    a = eng.generate(prompts, 12, loop="host", use_graph=True)
    b = eng.generate(prompts, 12, loop="device", use_graph=True)
    c = eng.generate(prompts, 12, loop="host", use_graph=False)
    assert _hash(a) == _hash(b) == _hash(c)
    assert all(len(o) == 12 for o in a)
    assert eng.last_stats["launches_per_step"] == 0 or eng.launches_per_step > 0

    # logits of the last prompt token vs stock PyTorch (same weights, not interleaved)
    wt = shard_for_rank(cfg, src, 0, 1, dev, interleave_gate_up=False)
    base = TorchLlamaTP(cfg, 0, 1, wt, dev, max_batch=1, max_seq_len=128)
    for p in prompts[:2]:
        eng.prefill([p], 1)
        got = eng.model.logits[:1].float().clone()
        ids = torch.tensor([p], device=dev)
        pos = torch.arange(len(p), device=dev, dtype=torch.int32)[None]
        with torch.no_grad():
            want = base.forward(ids, pos, 0)
        err = (got - want).abs().max().item()
        assert err < 0.05 * want.abs().max().item() + 0.02, err


def test_chunked_prefill_equals_single_chunk():
    from libtbvcoll_b200.engine.engine import Engine
    from libtbvcoll_b200.models.config import get_config
    cfg = get_config("tiny")
    dev = "cuda:0"
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (50, 33)]
    big = Engine(cfg, device=dev, seed=5, max_batch=2, max_seq_len=128, prefill_chunk=128)
    small = Engine(cfg, device=dev, seed=5, max_batch=2, max_seq_len=128, prefill_chunk=32)   # sequences straddle chunks
    assert big.generate(prompts, 6) == small.generate(prompts, 6)


def test_safetensors_checkpoint_round_trip(tmp_path):
    from libtbvcoll_b200.engine.engine import Engine
    from libtbvcoll_b200.models.config import get_config
    from libtbvcoll_b200.utils.weights import RandomSource, SafetensorsSource, save_hf_checkpoint
    cfg = get_config("tiny")
    dev = "cuda:0"
    src = RandomSource(cfg, seed=9, device="cpu")
    save_hf_checkpoint(src, str(tmp_path), max_shard_bytes=2 << 20)
    prompts = [[1, 2, 3, 4, 5, 6, 7]]
    a = Engine(cfg, device=dev, source=RandomSource(cfg, seed=9, device="cpu"), max_batch=1, max_seq_len=64, prefill_chunk=16).generate(prompts, 5)
    b = Engine(cfg, device=dev, source=SafetensorsSource(str(tmp_path)), max_batch=1, max_seq_len=64, prefill_chunk=16).generate(prompts, 5)
    assert a == b


@pytest.mark.parametrize("mode", ["2", "3"])
def test_long_prefill_through_the_many_token_gemm(persist_mode, mode):
    """A 448-row prefill chunk sends every plain and SiLU-mul GEMM through the persistent many-token kernel
    (TBV_GEMM_PERSIST=2: 128-token tiles, 3: 256-token tiles) inside the engine (strided activations, programmatic dependent launch); the logits
    must agree with the same prefill on the decode-form kernel."""
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.engine.engine import Engine
    from libtbvcoll_b200.models.config import get_config
    cfg = get_config("tiny")
    dev = "cuda:0"
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (400, 48)]
    eng = Engine(cfg, device=dev, seed=11, max_batch=2, max_seq_len=480, prefill_chunk=448)
    persist_mode(0)
    first_a = eng.prefill(prompts, 4)
    logits_a = eng.model.logits[:2].float().clone()
    persist_mode(int(mode))
    first_b = eng.prefill(prompts, 4)
    logits_b = eng.model.logits[:2].float().clone()
    torch.cuda.synchronize()
    assert not ops.gemm_error()
    err = (logits_a - logits_b).abs().max().item()
    assert err <= 0.02 * logits_a.abs().max().item() + 0.02, err
    assert len(first_a) == len(first_b) == 2


def test_captured_decode_loop_replayed_past_the_reserved_length():
    """The device-side decode loop keeps no host in it, so nothing but the kernels can stop it at the end
    of the reserved cache: the advance kernel stops the context length at the block table's capacity and
    hands out slot -1 (no cache write), and attention clamps the same way.  Replaying well past the
    capacity must neither read outside the block table nor disturb the run: tokens stay valid ids."""
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.engine.engine import Engine
    from libtbvcoll_b200.models.config import get_config
    cfg = get_config("tiny")
    eng = Engine(cfg, device="cuda:0", seed=3, max_batch=2, max_seq_len=32, block_size=16, prefill_chunk=16)
    prompts = [[1, 2, 3, 4, 5, 6, 7, 8], [9, 10, 11]]
    first = eng.prefill(prompts, 8)
    eng._load_decode_inputs(2, first, [len(p) for p in prompts])
    eng.step_counter.zero_()
    g = eng.capture(2, 1, True)
    cap = eng.bm.tables.shape[1] * eng.block_size
    for _ in range(cap + 9):                      # runs past position `cap`
        g.replay()
    torch.cuda.synchronize()
    assert not ops.gemm_error()
    assert int(eng.ctx[:2].max()) == cap           # clamped, not cap + 9
    assert int(eng.slots[:2].max()) == -1          # no cache slot past the table
    toks = eng.out_tokens[:2].tolist()
    assert all(0 <= t < cfg.vocab_size for t in toks)
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
