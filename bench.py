#!/usr/bin/env python
"""Headline benchmark: asynchronous GRPO steps on the Qwen2.5-1.5B architecture.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 2 --warmup 3

One step = one macro-batch of the full pipeline through the public ``Orchestrator`` API: rollout
(native engine) -> verifier rewards + group advantages -> old-policy logprobs -> packed microbatches ->
fused-loss forward/backward with gradient accumulation -> clipped AdamW step -> weight push to the logprob
and rollout roles. Workload (random-init weights, synthetic prompts): 16 prompts per GPU per step with
lengths uniform in [64, 512], 8 samples per prompt, generation lengths log-uniform in [256, 8192] with
EOS forced at the drawn length, Bernoulli(0.3) reward, packed microbatches of at most 32k tokens.
Per-GPU work is fixed as N grows (weak scaling); at N = 8 the placement is 4 trainer + 1 logprob +
3 rollout ranks and the step is 128 prompts x 8 samples.

Rank 0 prints one JSON line. ``--impl reference`` runs the same workload through the reference's own workers
(``baseline/reference_arm.py``).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen2.5-1.5b")
    ap.add_argument("--prompts-per-gpu", type=int, default=16)
    ap.add_argument("--samples-per-question", type=int, default=8)
    ap.add_argument("--gen-min", type=int, default=256)
    ap.add_argument("--gen-max", type=int, default=8192)
    ap.add_argument("--prompt-min", type=int, default=64)
    ap.add_argument("--prompt-max", type=int, default=512)
    ap.add_argument("--max-tokens-per-gpu", type=int, default=32768)
    ap.add_argument("--max-num-seqs", type=int, default=512)
    ap.add_argument("--preset", default="throughput", choices=["eager", "throughput"])
    ap.add_argument("--param-sharding", default="zero2", choices=["zero2", "zero3"],
                    help="zero3: fully sharded trainers (all-gather / reduce-scatter fused into the GEMM kernels)")
    ap.add_argument("--colocated-sm-limit", type=int, default=0,
                    help="SMs that trainer / logprob GEMMs may fill on a GPU shared with a rollout engine (0 = all)")
    ap.add_argument("--eager-dispatch", type=int, default=1,
                    help="1: finished samples go to the trainer at once (overlaps training with generation); 0: the trainer "
                         "starts when the minibatch is complete (the two measured the same on one GPU: 5.08 vs 4.98 samples/s)")
    ap.add_argument("--stream-logprobs", type=int, default=1)
    ap.add_argument("--colocated-rollout-sms", type=int, default=None,
                    help="SMs that the rollout engine gets for itself on a GPU it shares with other roles (default 0 = no "
                         "partition: measured slower on the one-GPU configuration, 29.5 s per step with 96 + 52 SMs against 25.3 s)")
    ap.add_argument("--generation-tp-size", type=int, default=1,
                    help="consecutive rollout ranks that form one tensor-parallel engine replica (1 = every rank a replica)")
    ap.add_argument("--placement", default=None, help='JSON role placement overriding the default, e.g. '
                    '\'{"trainer": [0, 1], "logprob": [0], "rollout": [1]}\'')
    # reference arm only (its own defaults: orchestrator.py:137, 158 of the reference)
    ap.add_argument("--ref-max-num-seqs", type=int, default=512, help="vLLM max_num_seqs of the reference arm (its default)")
    ap.add_argument("--ref-loss-chunksize", type=int, default=None, help="loss_chunksize of the reference arm (its default: none)")
    ap.add_argument("--ref-colocated-mem", type=float, default=0.10,
                    help="vLLM gpu_memory_utilization where the engine shares a GPU with FSDP workers (0.90 otherwise)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "500"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> None:
    """Runs the unmodified reference workers from ``baseline/_ref`` (see ``baseline/reference_arm.py``); every rank
    takes part, rank 0 prints the JSON line. Must be entered before ``torch`` is imported (it pins one GPU per process)."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not (os.path.isdir(ref_dir) and os.path.exists(os.path.join(ref_dir, "gpu_process_worker.py"))):
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref does not hold the reference tree (copy the "
                              "reference's *.py files there; pip cannot install it: no setup.py / pyproject.toml)"}))
        return
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as arm

    arm.run(args)


def placement_for(n: int):
    """Role placement per GPU count; roles share a GPU where there are fewer GPUs than roles."""
    if n == 1:
        return {"trainer": [0], "logprob": [0], "rollout": [0]}
    if n == 2:
        return {"trainer": [0], "logprob": [0], "rollout": [1]}
    if n == 4:
        return {"trainer": [0, 1], "logprob": [1], "rollout": [2, 3]}
    if n == 8:
        return {"trainer": [0, 1, 2, 3], "logprob": [4], "rollout": [5, 6, 7]}
    t = max(1, n // 2)
    return {"trainer": list(range(t)), "logprob": [t - 1], "rollout": list(range(t, n))}


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch

    from async_grpo_nccl_b200.config import make_config
    from async_grpo_nccl_b200.data import synthetic_prompt_rows
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.orchestrator import Orchestrator

    n = args.gpus
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != n and not (n == 1 and world == 1):
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n}")
    mcfg = PRESETS[args.model]
    prompts_per_step = args.prompts_per_gpu * n
    spq = args.samples_per_question
    total_steps = args.warmup + args.steps
    place = json.loads(args.placement) if args.placement else placement_for(n)
    cfg = make_config({
        "param_sharding": args.param_sharding, "colocated_sm_limit": args.colocated_sm_limit,
        "colocated_rollout_sms": int(args.colocated_rollout_sms or 0),
        "model_name_or_path": args.model, "batch_size": prompts_per_step, "samples_per_question": spq, "num_epochs": 1,
        "train_minibatch_sample_size": prompts_per_step * spq, "max_generation_tokens": args.gen_max,
        "max_tokens_per_gpu": args.max_tokens_per_gpu, "reward_fns": ["bernoulli"], "global_num_verifiers": 0,
        "num_training_gpu_workers": len(place["trainer"]), "num_logprob_gpu_workers": len(place["logprob"]),
        "num_generation_gpu_workers": len(place["rollout"]), "generation_tp_size": args.generation_tp_size, "placement": place, "learning_rate": 1e-6, "kl_beta": 0.001,
        "max_num_seqs": args.max_num_seqs, "vllm_engine_preset": args.preset, "eval_at_start": False, "temperature": 1.0,
        "min_samples_per_checkpoint": 10 ** 12, "seed": 0, "stream_logprobs": bool(args.stream_logprobs),
        "eager_microbatch_dispatch": bool(args.eager_dispatch),
    })
    rows = synthetic_prompt_rows(prompts_per_step * total_steps, mcfg.vocab_size, args.prompt_min, args.prompt_max, seed=0,
                                 samples_per_question=spq, gen_len_range=(args.gen_min, args.gen_max), reward_p=0.3)

    if n == 1:
        from async_grpo_nccl_b200.launch import build_inprocess_runtime

        runtime = build_inprocess_runtime(cfg, device="cuda:0")
        dist = None
    else:
        from async_grpo_nccl_b200.launch import build_distributed_runtime

        runtime = build_distributed_runtime(cfg)
        dist = runtime.dist

    result = run_timed(cfg, runtime, rows, args, n, rank, dist, mcfg)
    if rank == 0 and result is not None:
        print(json.dumps(result))


def run_timed(cfg, runtime, rows, args, n, rank, dist, mcfg):
    """Runs warm-up + timed macro-batches. Non-zero ranks serve their roles until rank 0 finishes."""
    import asyncio

    import torch

    from async_grpo_nccl_b200.orchestrator import Orchestrator, configure_logging

    configure_logging()
    if rank != 0:
        runtime.serve_forever()
        return None
    orch = Orchestrator(cfg, runtime=runtime, dataset=rows)
    sampler = ClockSampler()
    state = {}

    async def body():
        await runtime.initialize(orch)
        em = runtime.experience_manager
        for r in runtime.trainer_ranks:
            em.register_training_process(r, cfg.max_tokens_per_gpu, cfg.train_minibatch_sample_size)
        await runtime.start_trainers()
        bs = cfg.batch_size
        from async_grpo_nccl_b200.orchestrator import stamp_uids

        data = stamp_uids(rows)
        for i in range(args.warmup):
            await orch._run_macro_batch(data[i * bs:(i + 1) * bs], 0)
        # ---- timed region: barrier + synchronize on both sides, CUDA events on every rank ----
        await runtime.barrier_and_sync()
        before = await runtime.collect_stats()
        sampler.start()
        await runtime.record_event("start")
        t0 = time.time()
        recs = []
        for i in range(args.warmup, args.warmup + args.steps):
            recs.append(await orch._run_macro_batch(data[i * bs:(i + 1) * bs], 0))
        await runtime.record_event("stop")
        await runtime.barrier_and_sync()
        wall = time.time() - t0
        state["clocks"] = sampler.stop()
        state["device_ms"] = await runtime.elapsed_ms("start", "stop")  # max over ranks
        state["wall"] = wall
        state["recs"] = recs
        state["stats"] = (before, await runtime.collect_stats())
        await runtime.shutdown()

    asyncio.run(body())
    recs = state["recs"]
    samples = sum(int(r["training/batch_total_samples"]) for r in recs)
    gen_tokens = sum(float(r["generation/total_tokens_generated"]) for r in recs)
    dev_s = state["device_ms"] / 1000.0
    before, after = state["stats"]
    diff = {k: after.get(k, 0.0) - before.get(k, 0.0) for k in after}
    sync_ms = [float(r.get("timing/weight_sync_ms", 0.0)) for r in recs]
    sync_dev_ms = [float(r.get("timing/weight_sync_device_ms", 0.0)) for r in recs]
    place = cfg.resolved_placement()
    par = f"trainer{len(place['trainer'])}+logprob{len(place['logprob'])}+rollout{len(place['rollout'])}" + (" colocated" if n < 3 else "")
    out = {
        "metric": "GRPO samples/sec (gen tokens/sec and weight-sync ms in extra)",
        "value": samples / dev_s, "unit": "samples/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": state["device_ms"] / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random-init weights, random-token prompts, forced generation lengths)",
        "config": {"model": f"{args.model} architecture", "global_batch": cfg.batch_size * cfg.samples_per_question,
                   "prompts_per_step": cfg.batch_size, "samples_per_prompt": cfg.samples_per_question,
                   "seq_len": f"prompt U[{args.prompt_min},{args.prompt_max}] + generation logU[{args.gen_min},{args.gen_max}]",
                   "parallelism": par, "max_tokens_per_microbatch": cfg.max_tokens_per_gpu,
                   "l2": "working set (3.1 GB of weights, multi-GB KV cache and activations per step) is far larger than the 126 MB L2; no flush needed",
                   "engine_preset": cfg.vllm_engine_preset, "max_num_seqs": cfg.max_num_seqs,
                   "eager_microbatch_dispatch": bool(cfg.eager_microbatch_dispatch), "param_sharding": cfg.param_sharding, "generation_tp_size": cfg.generation_tp_size,
                   "colocated_rollout_sms": cfg.colocated_rollout_sms},
        "clocks": state["clocks"],
        "e2e": {"value": samples / state["wall"], "unit": "samples/s",
                "h2d_bytes_per_step": diff.get("h2d_bytes", 0.0) / args.steps, "d2h_bytes_per_step": diff.get("d2h_bytes", 0.0) / args.steps,
                "note": "host wall clock around the same macro-batches through Orchestrator; inputs are packed on the host into "
                        "pinned buffers and copied per microbatch, results (loss statistics, logprobs, generated ids) are read back"},
        "gpu_launches": int(diff.get("launches", 0.0)),
        "extra": {"gen_tokens_per_s": gen_tokens / dev_s, "weight_sync_ms_mean": sum(sync_ms) / max(1, len(sync_ms)),
                  "weight_sync_device_ms_mean": sum(sync_dev_ms) / max(1, len(sync_dev_ms)),
                  "samples": samples, "gen_tokens": gen_tokens, "optimizer_steps": sum(r["training/optimizer_steps_in_batch"] for r in recs),
                  # host seconds of the rollout engines' step loops inside the timed region, summed over engines
                  "engine_host": {k: round(v, 4) for k, v in diff.items() if k.startswith("engine_")}},
    }
    return out


if __name__ == "__main__":
    main()
