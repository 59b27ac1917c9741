#!/usr/bin/env python3
"""Headline benchmark: tensor-parallel greedy decode tokens/s of a Llama-3-8B-shaped model
(random-init bf16, batch 8, prompt 512 random token ids), one process per GPU.

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 2 --steps 64 --warmup 8

The quantity is the reference's headline (vLLM TP decode tok/s with its all-reduce hooked in,
step3b/vllm_tp_bench.py:165-209; published 170.9 tok/s at batch 8 on 2 laptops,
reports/10_tp_custom_allreduce.md:480).  Arms:
  --impl ours       this repository's engine (sm_100a kernels + tbvcoll collectives)   [default]
  --impl nccl       the path being replaced: stock PyTorch (cuBLAS) + NCCL all-reduce, CUDA-graphed
  --impl reference  the unmodified reference: HIP + Thunderbolt ibverbs, cannot exist on this box
Rank 0 prints ONE JSON line.  With 2 or more GPUs the line of ``--impl ours`` also carries
  nccl_same_engine   the SAME engine and kernels with every collective sent to torch.distributed (NCCL at its
                     default settings) and the plain add+RMSNorm operator — the reference's own experiment
                     (one engine, the all-reduce swapped: step3b/vllm_tp_bench.py:119-124);
  p50_allreduce_us   all-reduce latency at decode sizes (8 KB, 64 KB, 256 KB; bf16), this library against NCCL,
                     device time of calls captured in one CUDA graph, max over ranks, bit-exactness asserted.
``--shard-of N`` (one GPU): rank 0's shard of a TP=N model with every collective replaced by its local
arithmetic — no communication, wrong values; it exists to attribute the compute part of a TP=N step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REF_TOK_S_BATCH8 = 170.9   # reports/10_tp_custom_allreduce.md:480 (vLLM TP=2 + libtbvcoll, Qwen2.5-7B, 2x gfx1151)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl", "reference"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the end-to-end arm (0 = --steps, but at least 64)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the line INVALID)")
    ap.add_argument("--repeats", type=int, default=0, help="timed regions of --steps steps each (0 = enough for about 0.5 s in total, at most 12)")
    ap.add_argument("--shard-of", type=int, default=0, help="attribution only (marks the line INVALID): one GPU runs one rank's shard of a TP=N model, collectives replaced by local arithmetic")
    ap.add_argument("--no-extras", action="store_true", help="skip the same-engine NCCL arm and the all-reduce latencies")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of this rank's GPU, sampled every 50 ms; started a few
    periods before the timed region so that the region itself is covered."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            time.sleep(0.3)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max((float(r[2]) for r in self.rows if len(r) > 2 and r[2].replace('.', '', 1).isdigit()), default=None),
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    # The one offline pip install of the reference tree was attempted once and refused: "Directory is not
    # installable. Neither 'setup.py' nor 'pyproject.toml' found."  Its only build recipe is `hipcc --offload-arch=gfx1151 ... -libverbs` (README.md:6-7): no hipcc, no
    # libibverbs, no AMD GPU and no Thunderbolt RDMA device exist on a B200 box.
    here = os.path.dirname(os.path.abspath(__file__))
    if os.path.exists(os.path.join(here, "baseline", "_ref", "libtbvcoll.so")):
        why = "baseline/_ref holds a library but it targets gfx1151 + ibverbs and cannot load on a CUDA box"
    else:
        why = ("reference is HIP (gfx1151) + Thunderbolt ibverbs with no setup.py/pyproject: pip install refuses it, "
               "and hipcc/libibverbs/the tbv RDMA device do not exist on a B200 box")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def setup_dist(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs one process per GPU: launch with python -m torch.distributed.run "
                             f"--nnodes=1 --nproc-per-node {args.gpus} --master-addr 127.0.0.1 --master-port P bench.py ...")
        raise SystemExit(f"WORLD_SIZE={world} but --gpus {args.gpus}")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def max_over_ranks(x: float, world: int) -> float:
    import torch
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    import torch
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def timed_replays(replay, steps, warmup, world, repeats=1):
    """W untimed replays, then `repeats` timed regions of EXACTLY K replays each, every region bracketed
    by barrier + synchronize on both sides; device time by CUDA events, max over ranks.  Returns the
    list of ms per step, one per region."""
    import torch
    for _ in range(warmup):
        replay()
    out = []
    for _ in range(max(1, repeats)):
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            replay()
        e1.record()
        torch.cuda.synchronize()
        barrier(world)
        out.append(max_over_ranks(e0.elapsed_time(e1), world) / steps)
    return out


def decode_arm(eng, prompts, new_tokens, B, L, args, world, repeats, sampler=None):
    """Prefill, capture the decode step with the device-side feedback kernel, time it."""
    import torch
    first = eng.prefill(prompts, new_tokens)
    torch.cuda.synchronize()
    t_pf = time.perf_counter()
    first = eng.prefill(prompts, new_tokens)
    torch.cuda.synchronize()
    prefill_ms = max_over_ranks((time.perf_counter() - t_pf) * 1e3, world)
    splits = eng.attn_splits_for(B, L + new_tokens)
    eng._load_decode_inputs(B, first, [L] * B)
    eng.step_counter.zero_()
    graph = eng.capture(B, splits, True)
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    ms_all = timed_replays(graph.replay, args.steps, args.warmup, world, repeats)
    clocks = sampler.stop() if sampler is not None else None
    return ms_all, prefill_ms, splits, clocks


def allreduce_latencies(comm, world):
    """p50 device latency (us) of one all-reduce at decode sizes, this library (auto) and NCCL: 20 calls
    captured in one CUDA graph, median over 15 replays, max over ranks; this library's result is
    compared bit for bit with the fixed-order fp32 oracle first."""
    import torch
    import torch.distributed as dist
    from libtbvcoll_b200.bench_allreduce import graph_us
    rank = dist.get_rank()
    out = {}
    for nbytes in (8192, 65536, 262144):
        n = nbytes // 2
        xs = [torch.randn(n, generator=torch.Generator().manual_seed(4000 + r)).to(torch.bfloat16).cuda() for r in range(world)]
        acc = xs[0].float()
        for t in xs[1:]:
            acc = acc + t.float()
        want, x = acc.to(torch.bfloat16), xs[rank]
        y = torch.empty_like(x)
        if not comm.all_reduce(x, y):
            continue
        torch.cuda.synchronize()
        exact = bool(torch.equal(y, want))
        ours = graph_us(lambda: comm.all_reduce(x, y), 20, world)
        z = x.clone()
        nccl = graph_us(lambda: dist.all_reduce(z), 20, world)
        out[str(nbytes)] = {"ours": round(ours, 2), "nccl": round(nccl, 2), "bit_exact_vs_fixed_order_oracle": exact}
        if not exact:
            raise SystemExit(f"all-reduce of {nbytes} bytes is not bit-exact")
    return out


def run_ours(args, rank, world, local):
    import torch
    from libtbvcoll_b200 import ops
    from libtbvcoll_b200.engine.engine import Engine
    from libtbvcoll_b200.models.config import get_config
    from libtbvcoll_b200.parallel.tp import TPGroup
    from libtbvcoll_b200.tbvcoll import Comm
    cfg = get_config(args.model)
    if args.layers:
        cfg.num_layers = args.layers
    B, L = args.batch, args.prompt_len
    # end-to-end window: at least 64 steps, because the ten or so steps that follow a prefill run 4-5 % slower (the GPU is still
    # at the clocks its power cap allowed during the prefill GEMMs) and a 20-step window would mostly measure that
    e2e_steps = args.e2e_steps or max(args.steps, 64)
    repeats = args.repeats or max(1, min(12, -(-250 // max(1, args.steps))))     # about 250 timed steps in total
    new_tokens = max(256, args.steps * repeats + args.warmup + 2, e2e_steps + 2)
    chunk = 2048 if world > 1 else 4096       # prefill rows per forward pass (bounds the collective slot size when world > 1)
    comm = None
    if world > 1:
        port = int(os.environ.get("MASTER_PORT", "29500")) + 101
        comm = Comm(rank, world, local, os.environ.get("MASTER_ADDR", "127.0.0.1"), port, cap_bytes=chunk * cfg.hidden_size * 2)
    if args.shard_of > 1:
        assert world == 1, "--shard-of runs on one GPU"
        tp = TPGroup(0, args.shard_of, None, local_stand_in=True)
    else:
        tp = TPGroup(rank, world, comm)
    eng = Engine(cfg, tp, device=f"cuda:{local}", seed=0, max_batch=B, max_seq_len=L + new_tokens + 16, prefill_chunk=chunk)
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab_size, (L,), generator=g).tolist() for _ in range(B)]

    # ---- device-timed decode steps: the captured step replayed back to back (device loop) ----
    torch.cuda.synchronize()
    ms_all, prefill_ms, splits, clocks = decode_arm(eng, prompts, new_tokens, B, L, args, world, repeats, ClockSampler(local))
    ms = statistics.median(ms_all)
    value = B / (ms * 1e-3)
    phases = None
    if comm is not None:
        # per-phase device times of the collectives of the last replayed steps, every rank's stamps compared call by call
        from libtbvcoll_b200.bench_allreduce import trace_breakdown
        phases = trace_breakdown(comm, calls=1024)

    # ---- end to end through the public API: Engine.generate, host loop ----
    eng.generate(prompts, 4)                       # warm the host-loop graph
    barrier(world)
    eng.generate(prompts, e2e_steps + 1)
    e2e = B * e2e_steps / max_over_ranks(eng.last_stats["decode_s"], world)
    fallbacks = tp.fallbacks
    invalid = ("" if not args.layers else f"-INVALID-{args.layers}-layers") + ("" if args.shard_of <= 1 else f"-INVALID-shard-of-tp{args.shard_of}-no-communication")
    out = {
        "metric": "tp_decode_tokens_per_s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(value / REF_TOK_S_BATCH8, 2), "dtype": "bf16", "data": "synthetic (random token ids, random-init weights)",
        "impl": "ours",
        "config": {"model": cfg.name + invalid, "global_batch": B, "seq_len": L,
                   "decode_context": f"{L}..{L + args.steps * repeats + args.warmup}", "parallelism": f"tp{world}",
                   "l2": "inputs larger than L2: every step streams the rank's full weight shard "
                         f"({cfg.param_count() * 2 / world / 1e9:.1f} GB) from HBM",
                   "timing": f"CUDA events around K graph replays, max over ranks; {repeats} such regions back to back "
                             "(each bracketed by barrier + synchronize), value = median region",
                   "attn_splits": splits},
        "timed_regions_ms_per_step": [round(m, 4) for m in ms_all], "ms_per_step_min": round(min(ms_all), 4),
        "clocks": clocks,
        "e2e": {"value": round(e2e, 2), "unit": "tokens/s", "h2d_bytes_per_step": eng.h2d_bytes_per_step, "d2h_bytes_per_step": eng.d2h_bytes_per_step,
                "steps": e2e_steps, "api": "Engine.generate(prompts, max_new_tokens) host loop: per step the packed ids/slots/positions/"
                                           "context lengths are written to pinned memory, one graph launch copies them to the device, "
                                           "runs the step and copies the sampled tokens back to pinned memory, the host waits and reads them"},
        "gpu_launches": eng.launches_per_step * args.steps,
        "launches_per_step": eng.launches_per_step,
        "collective_fallbacks_to_nccl": fallbacks,
        "fused_gemm_allreduce": bool(world > 1 and tp.fuse_gemm),
        "prefill": {"ms": round(prefill_ms, 2), "tokens": B * L, "tokens_per_s": round(B * L / (prefill_ms * 1e-3), 1),
                    "sequence_parallel_chunks": eng.sp_chunks, "note": "wall clock with synchronize, second call, not part of the metric"},
        "baseline_note": "vs_baseline divides by the reference's published 170.9 tok/s (Qwen2.5-7B, vLLM TP=2, 2x gfx1151 laptops)",
    }
    if comm is not None:
        # the library's own device time stamps of the collectives of the last replays (kernel entry -> all peers' data seen -> done)
        _, wait_us, reduce_us, _, _, n_coll = comm.stats5()
        out["collective_device_us"] = {"wait_for_peers": round(wait_us, 2), "reduce_and_norm": round(reduce_us, 2), "calls_sampled": int(n_coll),
                                       "phases_all_ranks": phases}
    if world > 1 and not args.no_extras:
        # the same engine (same weights, same kernels) with the collectives on NCCL at its default settings
        tp_n = TPGroup(rank, world, None)
        eng_n = Engine(cfg, tp_n, device=f"cuda:{local}", weights=eng.model.w, max_batch=B, max_seq_len=L + new_tokens + 16, prefill_chunk=chunk)
        ms_n, _, _, _ = decode_arm(eng_n, prompts, new_tokens, B, L, args, world, min(repeats, 3))
        m = statistics.median(ms_n)
        out["nccl_same_engine"] = {"ms_per_step": round(m, 4), "value": round(B / (m * 1e-3), 2), "unit": "tokens/s",
                                   "launches_per_step": eng_n.launches_per_step, "nccl_calls_per_step": 2 * cfg.num_layers + 2,
                                   "what": "this engine and its kernels; all-reduce / all-gather by torch.distributed (NCCL defaults, "
                                           "captured in the same CUDA graph), then the plain add+RMSNorm operator"}
        out["ours_over_nccl_same_engine"] = round(m / ms, 3)
        del eng_n
        out["p50_allreduce_us"] = allreduce_latencies(comm, world)
    if comm is not None:
        comm.destroy()
    return out


def run_nccl(args, rank, world, local):
    """Stock PyTorch TP decode step (cuBLAS + NCCL), CUDA-graphed; same shape, same timing rules."""
    import torch
    from libtbvcoll_b200.models.config import get_config
    from libtbvcoll_b200.models.torch_baseline import GraphedTorchDecoder, TorchLlamaTP
    from libtbvcoll_b200.utils.weights import RandomSource, shard_for_rank
    cfg = get_config(args.model)
    if args.layers:
        cfg.num_layers = args.layers
    B, L = args.batch, args.prompt_len
    dev = f"cuda:{local}"
    w = shard_for_rank(cfg, RandomSource(cfg, seed=0, device=dev), rank, world, dev, interleave_gate_up=False)
    m = TorchLlamaTP(cfg, rank, world, w, dev, max_batch=B, max_seq_len=L + 64)
    with torch.no_grad():
        g = torch.Generator().manual_seed(1234)
        prompts = torch.stack([torch.randint(0, cfg.vocab_size, (L,), generator=g) for _ in range(B)]).to(dev)
        pos = torch.arange(L, device=dev, dtype=torch.int32)[None].expand(B, L)
        m.forward(prompts, pos, 0)
        dec = GraphedTorchDecoder(m, B, L)
        dec.pos.fill_(L)
        dec.capture()
    sampler = ClockSampler(local)
    sampler.start()
    ms = statistics.median(timed_replays(dec.replay, args.steps, args.warmup, world, 3))
    clocks = sampler.stop()
    value = B / (ms * 1e-3)
    return {"metric": "tp_decode_tokens_per_s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / REF_TOK_S_BATCH8, 2), "dtype": "bf16", "data": "synthetic",
            "impl": "nccl+cublas (plain PyTorch ops, unoptimised: unfused norm/RoPE, mask-path attention)",
            "config": {"model": cfg.name, "global_batch": B, "seq_len": L, "parallelism": f"tp{world}",
                       "note": "fixed context of prompt_len+1 per step (static shapes under CUDA graph)"},
            "clocks": clocks, "gpu_launches": 0}


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    rank, world, local = setup_dist(args)
    out = run_ours(args, rank, world, local) if args.impl == "ours" else run_nccl(args, rank, world, local)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
