#!/usr/bin/env python3
"""vLLM tensor-parallel decode benchmark with the tbvcoll all-reduce hooked in.

Same shape as the reference's bench (step3b/vllm_tp_bench.py:142-209): an external-launcher
vLLM engine (one process per GPU under torchrun), greedy sampling with ``ignore_eos``, ``batch``
copies of one prompt with a per-copy suffix, a warm-up, then per round barrier -> generate ->
barrier; prints tokens/s per round and the sha256 of all generated token ids per round (the
output-hash gate: run once with ``--tbvcoll`` and once without and compare), then median / max
tokens/s and the hook's call / fallback counters.

There is no network on the benchmark hosts, so besides a real HF model directory the script can
synthesise one: ``--synth llama3-8b`` writes a config.json for that shape into a temp directory
and loads vLLM with dummy (random) weights and token-id prompts (no tokenizer).

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m libtbvcoll_b200.integrations.vllm_tp_bench \
        --synth llama3-8b --tp 2 --batch 8 --out-tokens 128 --tbvcoll
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import tempfile
import time


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="")
    ap.add_argument("--synth", default="", help="model preset to synthesise (dummy weights), e.g. llama3-8b")
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--out-tokens", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--gpu-mem-util", type=float, default=0.6)
    ap.add_argument("--compile", action="store_true", help="let vLLM compile / capture graphs (default: eager, like the reference)")
    ap.add_argument("--tbvcoll", action="store_true", help="hook GroupCoordinator.all_reduce")
    ap.add_argument("--tbv-eager", action="store_true", help="bring the library up before the engine sizes its KV cache")
    ap.add_argument("--time-nccl", action="store_true", help="per-call synchronised timing of the ORIGINAL all-reduce (invasive)")
    ap.add_argument("--dbo", action="store_true", help="accepted for parity; dual-batch overlap is not a goal here")
    ap.add_argument("--tbv-cap", type=int, default=4 << 20)
    ap.add_argument("--ar-fusion", default="auto", choices=["auto", "on", "off"],
                    help="--compile only: vLLM's own all-reduce + RMSNorm fusion pass (it compiles the TP all-reduce away, so a "
                         "hook on the all-reduce is never called).  auto = off with --tbvcoll, vLLM's default otherwise")
    return ap.parse_args()


def synth_model_dir(preset: str) -> str:
    from ..models.config import get_config
    c = get_config(preset)
    d = tempfile.mkdtemp(prefix=f"tbv-{preset}-")
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": c.hidden_size,
           "num_hidden_layers": c.num_layers, "num_attention_heads": c.num_heads, "num_key_value_heads": c.num_kv_heads,
           "head_dim": c.head_dim, "intermediate_size": c.intermediate_size, "vocab_size": c.vocab_size, "rope_theta": c.rope_theta,
           "rms_norm_eps": c.rms_eps, "max_position_embeddings": c.max_position, "hidden_act": "silu", "torch_dtype": "bfloat16",
           "tie_word_embeddings": c.tie_embeddings, "attention_bias": c.qkv_bias, "bos_token_id": 1, "eos_token_id": 2}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


def main():
    args = parse()
    os.environ.setdefault("TBV_CAP", str(args.tbv_cap))
    import torch
    import torch.distributed as dist
    from vllm import LLM, SamplingParams
    from . import vllm_hook
    if args.dbo:
        print("# --dbo: dual-batch overlap needs DP>1 in vLLM and was withdrawn as a goal by the reference "
              "(reports/11_custom_engine.md:121-151); ignored")
    if args.time_nccl:
        vllm_hook.install_nccl_timing()
    elif args.tbvcoll:
        # --tbv-eager: bring the library up NOW, before the engine exists, so that its slot memory is allocated
        # before vLLM sizes its KV cache (step3b/vllm_tp_bench.py:129-139); all ranks are at the same point
        vllm_hook.install(eager=args.tbv_eager)
    model = args.model or synth_model_dir(args.synth or "llama3-8b")
    dummy = not args.model
    extra = {}
    fusion_off = args.ar_fusion == "off" or (args.ar_fusion == "auto" and args.tbvcoll)
    if args.compile and fusion_off:
        # Under torch.compile current vLLM pattern-matches all_reduce + RMSNorm into its own fused kernel, after which the
        # TP all-reduce this benchmark is about no longer exists as a call.  Comparable runs switch the pass off on both sides.
        extra["compilation_config"] = {"pass_config": {"fuse_allreduce_rms": False}}
        print("# vLLM's all-reduce + RMSNorm fusion pass is OFF for this run (--ar-fusion)", flush=True)
    llm = LLM(model=model, tensor_parallel_size=args.tp, distributed_executor_backend="external_launcher",
              enforce_eager=not args.compile, seed=1, max_model_len=args.max_model_len, gpu_memory_utilization=args.gpu_mem_util,
              **({"load_format": "dummy", "skip_tokenizer_init": True} if dummy else {}), **extra)
    sp = SamplingParams(temperature=0.0, max_tokens=args.out_tokens, ignore_eos=True, **({"detokenize": False} if dummy else {}))
    if dummy:
        g = torch.Generator().manual_seed(1234)
        base = torch.randint(10, 30000, (args.prompt_len,), generator=g).tolist()
        prompts = [{"prompt_token_ids": base[:-1] + [100 + i]} for i in range(args.batch)]
    else:
        prompts = [f"Explain tensor parallelism in one paragraph. Variant {i}." for i in range(args.batch)]
    rank = dist.get_rank() if dist.is_initialized() else 0
    llm.generate(prompts, sp, use_tqdm=False)            # warm-up
    rates = []
    for r in range(args.rounds):
        dist.barrier()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp, use_tqdm=False)
        dist.barrier()
        dt = time.perf_counter() - t0
        ids = [list(o.outputs[0].token_ids) for o in outs]
        ntok = sum(len(x) for x in ids)
        h = hashlib.sha256(json.dumps(ids).encode()).hexdigest()[:16]
        rates.append(ntok / dt)
        if rank == 0:
            print(f"round {r}: {ntok} tokens in {dt:.3f}s = {ntok / dt:.1f} tok/s  hash={h}", flush=True)
    if rank == 0:
        print(f"median {statistics.median(rates):.1f} tok/s  max {max(rates):.1f} tok/s  batch={args.batch} tp={args.tp} "
              f"tbvcoll={int(args.tbvcoll)}")
        print(vllm_hook.summary())
        if args.tbvcoll:
            from .. import tbvcoll
            pre, xfer, post, enq, drain, n = tbvcoll.stats5()
            print(f"tbvcoll: {n} collectives, device wait-for-peers {xfer:.2f} us, reduce {post:.2f} us, host enqueue {enq:.2f} us")


if __name__ == "__main__":
    main()
