"""Reference arm of ``bench.py``: the reference's own code on the headline workload, on this box.

What runs unmodified from ``baseline/_ref`` (a plain copy of the reference tree; pip cannot install it, it has
no package metadata):

* ``gpu_process_worker.TrainerGPUWorker``: ``init_distributed_env``, ``init_model`` (HF ``from_pretrained``,
  FA2 varlen wrapper, ``make_grpo_forward``, ``fully_shard`` per block + root with its mixed-precision policy,
  AdamW + LambdaLR), ``compute_gradients`` (``post_process_batch`` + ``compute_dual_clip_grpo_loss`` + sample
  scaling + backward), ``apply_gradients`` (clip 1.0 + step), ``get_trainer_weights_info``, ``sync_weights``
  (``full_tensor()`` + one broadcast per tensor);
* ``gpu_process_worker.LogProbGPUWorker``: ``init_model``, ``compute_log_probs_from_samples``, ``sync_weights``;
* ``grpo_loss`` and ``sample_processing_utils`` underneath them.

What is restated here because its module cannot load without Ray actors / vLLM v0 (listed in the JSON line
under ``restated``): the config record (orchestrator.py:92-193), the per-prompt sample construction and group
advantages (vllm_worker.py:749-796), the logprob token-budget batcher (logprob_worker.py:144-216), the
microbatch planner (orchestrator.py:1892-2005), the rollout worker's receive loop (gpu_process_worker.py:
1888-1915) and the control plane (a TCP key-value store instead of Ray RPC). Generation runs in vLLM 0.22 with
the reference's engine arguments (vllm_worker.py:219-232), in the rollout rank's own process.

One process per GPU, one GPU per process (``CUDA_VISIBLE_DEVICES`` = local rank, as Ray isolates the
reference's actors). Nothing here imports ``async_grpo_nccl_b200``.
"""
from __future__ import annotations

import json
import os
import pickle
import sys
import threading
import time
from typing import Any, Dict, List, Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))

RESTATED = [
    "OrchestratorConfig fields (orchestrator.py:92-193)",
    "sample construction + group advantages (vllm_worker.py:749-796); one request per sample so that each sample gets its drawn length",
    "logprob token-budget batcher (logprob_worker.py:144-216)",
    "microbatch planner: least-token rank, dummy batches, GRADIENT_STEP (orchestrator.py:1892-2005)",
    "rollout receive loop: empty + broadcast + load_weights per tensor (gpu_process_worker.py:1888-1915)",
    "control plane: TCP store mailboxes instead of Ray RPC; vLLM's in-process executor instead of ExternalProcessExecutor",
]


def placement_for(n: int) -> Dict[str, List[int]]:
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


class RefConfig:
    """The attributes the reference's GPU workers read from ``OrchestratorConfig`` (orchestrator.py:92-193)."""

    def __init__(self, **kw: Any):
        self.model = {"path": kw["model_name_or_path"], "lora_rank": 0, "lora_alpha": 16, "target_modules": ["q_proj", "v_proj"],
                      "trust_remote_code": True}
        self.trainer = {"optim": {"lr": kw.get("learning_rate", 1e-6), "weight_decay": 0.0, "lr_warmup_steps": 0,
                                  "lr_scheduler": "constant", "total_training_steps": 0},
                        "fsdp": {"param_offload": False, "optimizer_offload": False}}
        self.clip_low = kw.get("clip_low", 0.2)
        self.clip_high = kw.get("clip_high", 0.28)
        self.clip_ratio_c = kw.get("clip_ratio_c", 3.0)
        self.temperature = kw.get("temperature", 1.0)
        self.train_minibatch_sample_size = kw["train_minibatch_sample_size"]
        self.max_tokens_per_gpu = kw.get("max_tokens_per_gpu", 36000)
        self.apply_entropy_bonus = True
        self.entropy_coeff = 0.0
        self.use_torch_compile = bool(kw.get("use_torch_compile", True))
        self.loss_chunksize = kw.get("loss_chunksize", None)
        self.max_num_seqs = kw.get("max_num_seqs", 512)
        self.enable_prefix_caching = True
        self.vllm_engine_preset = kw.get("vllm_engine_preset", "eager")


# ------------------------------------------------------------------------------------------------ control plane
class Mail:
    """Mailboxes on a TCP key-value store: ``post(box, obj)`` / ``take(box)`` in posting order per box. Payloads above
    1 MB (sample lists of a whole microbatch) travel as a file in a spool directory of this node and only the file name
    goes through the store, the way Ray keeps large arguments in its object store and sends references."""

    BIG = 1 << 20

    def __init__(self, store, spool: Optional[str] = None):
        self.store = store
        self.next: Dict[str, int] = {}
        self.spool = spool
        if spool:
            os.makedirs(spool, exist_ok=True)

    def post(self, box: str, obj: Any) -> None:
        idx = self.store.add(f"{box}/n", 1)
        data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        if self.spool and len(data) > self.BIG:
            path = os.path.join(self.spool, f"{box.replace('/', '_')}_{idx}.pkl")
            with open(path + ".tmp", "wb") as f:
                f.write(data)
            os.replace(path + ".tmp", path)
            data = b"FILE:" + path.encode()
        self.store.set(f"{box}/{idx}", data)

    def ready(self, box: str) -> bool:
        nxt = self.next.get(box, 1)
        return bool(self.store.check([f"{box}/{nxt}"]))

    def take(self, box: str) -> Any:
        nxt = self.next.get(box, 1)
        key = f"{box}/{nxt}"
        data = self.store.get(key)
        self.store.delete_key(key)
        self.next[box] = nxt + 1
        if data[:5] == b"FILE:":
            path = data[5:].decode()
            with open(path, "rb") as f:
                data = f.read()
            os.remove(path)
        return pickle.loads(data)

    def barrier(self, name: str, world: int) -> None:
        n = self.store.add(f"bar/{name}", 1)
        if n == world:
            self.store.set(f"bar/{name}/go", b"1")
        self.store.get(f"bar/{name}/go")


# ------------------------------------------------------------------------------------------------ planner (restated)
def plan_microbatches(samples: List[dict], trainer_ranks: int, max_tokens: int, minibatch: int) -> List[List[Tuple[str, Any]]]:
    """Per-trainer-rank message lists for one macro-batch, built the way the reference's ExperienceManager does
    (orchestrator.py:1892-2005): every sample goes to the rank holding the fewest tokens; a full rank flushes one
    MICROBATCH to every rank (a dummy where a rank is empty); reaching the minibatch size emits GRADIENT_STEP."""
    msgs: List[List[Tuple[str, Any]]] = [[] for _ in range(trainer_ranks)]
    batches: List[List[dict]] = [[] for _ in range(trainer_ranks)]
    lens = [0] * trainer_ranks
    sent = 0
    total_tokens = sum(s["num_non_masked_output_tokens"] for s in samples)

    def dispatch() -> int:
        n_real = sum(len(b) for b in batches)
        if n_real == 0:
            return 0
        for r in range(trainer_ranks):
            msgs[r].append(("microbatch", batches[r] if batches[r] else [{"dummy": True, "total_non_masked_output_tokens": 0}]))
            batches[r] = []
            lens[r] = 0
        return n_real

    for s in samples:
        s["total_non_masked_output_tokens"] = total_tokens
        n = s["input_len"] + s["output_len"]
        r = min(range(trainer_ranks), key=lambda i: lens[i])
        if lens[r] + n > max_tokens:
            sent += dispatch()
        batches[r].append(s)
        lens[r] += n
        if sent + sum(len(b) for b in batches) == minibatch:
            dispatch()
            for q in msgs:
                q.append(("gradient_step", None))
            sent = 0
    if dispatch():
        for q in msgs:
            q.append(("gradient_step", None))
    for q in msgs:
        q.append(("batch_done", None))
    return msgs


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines: List[str] = []

    def start(self):
        import subprocess
        import threading

        try:
            env = {k: v for k, v in os.environ.items() if k != "CUDA_VISIBLE_DEVICES"}
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "500"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, env=env)
            threading.Thread(target=lambda: [self.lines.append(ln.strip()) for ln in self.proc.stdout], daemon=True).start()
        except Exception:
            self.proc = None

    def stop(self) -> Dict[str, Any]:
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
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ roles
class RolloutRole:
    """vLLM 0.22 engine in this process with the reference's engine arguments (vllm_worker.py:219-232, 259-279)."""

    def __init__(self, cfg: RefConfig, mem_fraction: float, tokenizer):
        from vllm import LLM

        kw: Dict[str, Any] = dict(model=cfg.model["path"], tensor_parallel_size=1, gpu_memory_utilization=mem_fraction,
                                  dtype="bfloat16", enable_prefix_caching=cfg.enable_prefix_caching, max_num_seqs=cfg.max_num_seqs,
                                  max_model_len=32768, load_format="auto", disable_custom_all_reduce=True, disable_log_stats=True,
                                  trust_remote_code=True, seed=0)
        if cfg.vllm_engine_preset == "eager":
            kw["enforce_eager"] = True
        self.llm = LLM(**kw)
        self.engine = self.llm.llm_engine
        self.tokenizer = tokenizer
        self.temperature = cfg.temperature
        self.model = self._find_model()
        self.req = 0
        self.engine_steps = 0

    def _find_model(self):
        """The nn.Module inside vLLM's (in-process) worker, whose ``load_weights`` the reference calls per tensor."""
        def of_worker(w):
            w = getattr(w, "worker", w)
            return w.get_model() if hasattr(w, "get_model") else w.model_runner.model

        try:
            return self.llm.collective_rpc(of_worker)[0]
        except Exception:
            pass
        ex = getattr(self.engine, "model_executor", None) or getattr(getattr(self.engine, "engine_core", None), "engine_core", None)
        ex = getattr(ex, "model_executor", ex)
        return of_worker(getattr(ex, "driver_worker", None))

    def generate(self, rows: List[dict], on_group) -> Tuple[int, float]:
        """All samples of ``rows`` (one request per sample, each with its drawn length); ``on_group(samples)`` is
        called when the last sample of a prompt finishes."""
        from vllm import SamplingParams, TokensPrompt

        t0 = time.time()
        pending: Dict[str, Tuple[int, int]] = {}
        outs: Dict[int, Dict[int, List[int]]] = {}
        for gi, row in enumerate(rows):
            ids = [int(t) for t in row["input_token_ids"]]
            row["input_token_ids"] = ids
            outs[gi] = {}
            for c, L in enumerate(row["forced_output_lens"]):
                L = max(1, min(int(L), 32768 - len(ids) - 1))
                sp = SamplingParams(n=1, temperature=self.temperature, seed=c, max_tokens=L, min_tokens=L, ignore_eos=True,
                                    include_stop_str_in_output=True, spaces_between_special_tokens=False, skip_special_tokens=False,
                                    detokenize=False)
                rid = f"inference-{row['__uid__']}-{c}-{self.req}"
                self.req += 1
                pending[rid] = (gi, c)
                self.engine.add_request(rid, TokensPrompt(prompt_token_ids=ids), sp)
        total = 0
        while self.engine.has_unfinished_requests():
            self.engine_steps += 1
            for o in self.engine.step():
                if not o.finished:
                    continue
                gi, c = pending.pop(o.request_id)
                toks = list(o.outputs[0].token_ids)
                total += len(toks)
                outs[gi][c] = toks
                if len(outs[gi]) == len(rows[gi]["forced_output_lens"]):
                    on_group(self._build_group(rows[gi], outs.pop(gi)))
        return total, time.time() - t0

    def _build_group(self, row: dict, outs: Dict[int, List[int]]) -> List[dict]:
        import numpy as np
        from copy import deepcopy

        from ref_workload import bernoulli_reward

        eos = self.tokenizer.eos_token_id
        base = {k: v for k, v in row.items() if k != "forced_output_lens"}
        base["input_len"] = len(row["input_token_ids"])
        samples = []
        for c in sorted(outs):
            s = deepcopy(base)
            s["sample_index"] = c
            s["modified_reward"] = None
            s["delimiter_not_found"] = False
            s["output_token_ids"] = outs[c]
            s["output_token_ids"][-1] = eos  # EOS forced at the drawn length
            s["output_len"] = len(s["output_token_ids"])
            s["sample_ids"] = s["input_token_ids"] + s["output_token_ids"]
            s["sample_text"] = self.tokenizer.decode(s["sample_ids"])
            s["sample_position_ids"] = list(range(len(s["sample_ids"])))
            s["truncated_sample"] = (s["sample_ids"][-1] != eos)
            labels = [-100] * len(s["sample_ids"])
            for i in range(s["output_len"]):
                pos = s["input_len"] + i
                labels[pos] = s["sample_ids"][pos]
            s["labels"] = labels
            s["num_non_masked_output_tokens"] = sum(1 for lb in labels if lb != -100)
            s["reward"] = bernoulli_reward(s)
            s["reward_success"] = True
            samples.append(s)
        r = np.array([s["reward"] for s in samples])
        adv = (r - float(np.mean(r))) / float(np.std(r) + 1e-4)
        for s, a in zip(samples, adv):
            s["advantage"] = float(a)
        return samples

    def receive_weights(self, weights_info, group) -> None:
        import torch

        for key, shape, dtype in weights_info:
            tensor = torch.empty(shape, dtype=dtype, device="cuda")
            group.broadcast(tensor, 0, "sync_group")
            self.model.load_weights([(key, tensor)])


class LogprobBatcher:
    """Token-budget batching of logprob requests (logprob_worker.py:144-216): keep adding while the sum of sample
    lengths stays below the budget, wait 10 ms for one more, carry over the request that did not fit."""

    def __init__(self, worker, budget: int):
        self.worker, self.budget = worker, budget
        self.queue: List[dict] = []
        self.h2d = 0
        self.d2h = 0

    def run_ready(self, more_coming: bool, poll) -> List[dict]:
        if not self.queue:
            return []
        batch, tokens = [], 0
        while True:
            while self.queue and (not batch or tokens + len(self.queue[0]["sample_ids"]) < self.budget):
                s = self.queue.pop(0)
                batch.append(s)
                tokens += len(s["sample_ids"])
            if self.queue or not more_coming:
                break
            time.sleep(0.010)
            if not poll():
                break
        res = self.worker.compute_log_probs_from_samples(batch)
        for s, r in zip(batch, res):
            s["sample_logprobs"] = r["logprobs"]
            s["sample_entropies"] = r["entropies"]
        self.h2d += 3 * 8 * tokens
        self.d2h += 2 * 4 * tokens
        return batch


# ------------------------------------------------------------------------------------------------ main
# Where this rank currently is (name, start time): a watchdog ends the arm when one phase takes longer than the limit, so a
# deadlock between the reference's workers shows up as an `unavailable` line instead of an hour-long rendezvous timeout.
PHASE: Dict[str, Any] = {"name": "start", "t": time.time()}
PHASE_LIMIT_S = float(os.environ.get("AGRPO_REF_PHASE_LIMIT_S", "1200"))


def set_phase(name: str) -> None:
    PHASE["name"], PHASE["t"] = name, time.time()


def write_abort(path: str, msg: str) -> None:
    """Leaves a failure note for the other ranks of this run (first writer wins)."""
    try:
        fd = os.open(path, os.O_CREAT | os.O_EXCL | os.O_WRONLY, 0o644)
    except FileExistsError:
        return
    with os.fdopen(fd, "w") as f:
        f.write(msg)


def read_abort(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read() or "a rank of the reference arm failed"
    except FileNotFoundError:
        return None


def run(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29533"))
    n = args.gpus
    if world != n and not (n == 1 and world == 1):
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}")
    # One visible GPU per process (the reference's actors get theirs from Ray) and no launcher variables left for
    # vLLM or the workers to pick up; the workers' own RANK / WORLD_SIZE are set below per role group.
    os.environ["CUDA_VISIBLE_DEVICES"] = os.environ.get("CUDA_VISIBLE_DEVICES", ",".join(map(str, range(64)))).split(",")[local_rank]
    for k in list(os.environ):
        if k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_WORLD_SIZE",
                 "GROUP_WORLD_SIZE", "ROLE_NAME") or k.startswith("TORCHELASTIC_"):
            os.environ.pop(k)
    os.environ.update({"HF_HUB_OFFLINE": "1", "TRANSFORMERS_OFFLINE": "1", "VLLM_ENABLE_V1_MULTIPROCESSING": "0",
                       "VLLM_NO_USAGE_STATS": "1", "VLLM_DO_NOT_TRACK": "1", "TOKENIZERS_PARALLELISM": "false",
                       "VLLM_LOGGING_LEVEL": os.environ.get("VLLM_LOGGING_LEVEL", "WARNING"), "GRPO_LOGGING_LEVEL": "WARNING",
                       "LOCAL_RANK": "0"})
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.join(HERE, "_ref"))
    # A rank that fails must not leave the others in their rendezvous timeouts (minutes each): it drops a note that every
    # rank's watchdog thread looks for; rank 0 then reports `unavailable` and all of them leave at once.
    abort_path = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"agrpo_ref_abort_{port}_{os.getppid() if world > 1 else os.getpid()}")
    printed = threading.Lock()

    def report(msg: str) -> None:
        if rank == 0 and printed.acquire(blocking=False):
            print(json.dumps({"impl": "reference", "unavailable": msg[:400]}), flush=True)

    def watchdog() -> None:
        while True:
            time.sleep(2.0)
            msg = read_abort(abort_path)
            if msg is None and time.time() - PHASE["t"] > PHASE_LIMIT_S:
                msg = f"reference arm timed out on rank {rank} in phase '{PHASE['name']}' after {int(PHASE_LIMIT_S)} s"
                write_abort(abort_path, msg)
            if msg is not None:
                report(msg)
                if rank != 0 and world > 1:
                    time.sleep(5.0)  # let rank 0 print first
                os._exit(0)

    set_phase("start")
    threading.Thread(target=watchdog, name="abort-watchdog", daemon=True).start()
    result = None
    try:
        result = _run(args, rank, n, host, port)
    except Exception as e:  # the arm reports instead of failing the round's bench step
        import traceback

        traceback.print_exc()
        msg = f"reference arm failed on rank {rank}: {type(e).__name__}: {str(e)[:300]}"
        write_abort(abort_path, msg)
        report(msg)
        if rank != 0 and world > 1:
            time.sleep(5.0)  # rank 0's watchdog prints the line; this process must not be the first to vanish
        os._exit(0)
    if rank == 0 and result is not None and printed.acquire(blocking=False):
        print(json.dumps(result), flush=True)
    os._exit(0)  # vLLM and NCCL helper threads must not keep the process alive


def _run(args, rank: int, n: int, host: str, port: int) -> Optional[Dict[str, Any]]:
    import asyncio
    from datetime import timedelta

    import torch
    import torch.distributed as dist

    import ref_shims
    from ref_workload import ARCHS, build_model_dir, synthetic_rows

    shims = ref_shims.install()
    place = json.loads(args.placement) if getattr(args, "placement", None) else placement_for(n)
    T, L, R = place["trainer"], place["logprob"], place["rollout"]
    is_t, is_l, is_r = rank in T, rank in L, rank in R
    store = dist.TCPStore(host, port + 21, world_size=n, is_master=(rank == 0), timeout=timedelta(seconds=3600),
                          wait_for_workers=False)
    mail = Mail(store, spool=os.path.join(os.environ.get("TMPDIR", "/tmp"), f"agrpo_ref_mail_{port}"))
    torch.cuda.set_device(0)

    # ---- model directory (rank 0 writes it; same random-init weights for every role) ----
    set_phase("model directory")
    model_dir = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"agrpo_ref_{args.model}_{port}")
    if rank == 0:
        build_model_dir(model_dir, args.model, seed=0)
    mail.barrier("model_dir", n)

    arch = ARCHS[args.model]
    spq = args.samples_per_question
    prompts_per_step = args.prompts_per_gpu * n
    minibatch = prompts_per_step * spq
    cfg = RefConfig(model_name_or_path=model_dir, learning_rate=1e-6, temperature=1.0, train_minibatch_sample_size=minibatch,
                    max_tokens_per_gpu=args.max_tokens_per_gpu, max_num_seqs=args.ref_max_num_seqs, vllm_engine_preset=args.preset,
                    loss_chunksize=args.ref_loss_chunksize)
    from transformers import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(model_dir, trust_remote_code=True)

    # ---- rollout engine first: in a process that also hosts FSDP workers it creates the (single-rank) default
    # process group that those workers then find initialised ----
    set_phase("rollout engine start")
    rollout = None
    if is_r:
        colocated = is_t or is_l
        rollout = RolloutRole(cfg, args.ref_colocated_mem if colocated else 0.90, tokenizer)

    import gpu_process_worker as gpw

    ref_shims.retire()
    shims["transformers._no_split_modules"] = ref_shims.transformers_compat()
    set_phase("trainer / logprob worker start")
    trainer = logprob = None
    if is_t:
        os.environ["RANK"], os.environ["WORLD_SIZE"] = str(T.index(rank)), str(len(T))
        trainer = gpw.TrainerGPUWorker(cfg)
        asyncio.run(trainer.init_distributed_env(f"tcp://{host}:{port + 22}"))
        if n == 4 and len(L) == 1 and L[0] in T:
            # the logprob worker that shares a process with a trainer rank needs a group of its own for its barrier
            solo = dist.new_group(ranks=[T.index(L[0])])
        trainer.init_model(for_computation=True)
        trainer.load_own_initial_weights()
    if is_l:
        if not is_t:
            os.environ["RANK"], os.environ["WORLD_SIZE"] = "0", "1"
        logprob = gpw.LogProbGPUWorker(cfg)
        if is_t and len(T) > 1:
            logprob.rank, logprob.world_size, logprob.global_rank = 0, 1, 0
        else:
            asyncio.run(logprob.init_distributed_env(f"tcp://{host}:{port + 23 + L.index(rank)}"))
        logprob.init_model(for_computation=False, fsdp_group_ranks=[0] if (is_t and len(T) > 1) else None)
        if is_t and len(T) > 1:
            logprob.fsdp_group = solo
    # ---- the sync group: one member per process, order trainer + logprob + rollout ----
    set_phase("sync group")
    order = list(dict.fromkeys(T + L + R))
    group = ref_shims.SYNC_GROUP
    group.rank, group.world = order.index(rank), len(order)
    if len(order) > 1:
        from vllm.distributed.device_communicators.pynccl import PyNcclCommunicator
        from vllm.distributed.utils import StatelessProcessGroup

        pg = StatelessProcessGroup.create(host=host, port=port + 30, rank=group.rank, world_size=group.world)
        group.comm = PyNcclCommunicator(pg, device=torch.device("cuda:0"))
    weights_info = None
    if rank == T[0]:
        weights_info = [(k, tuple(s), d) for k, s, d in trainer.get_trainer_weights_info()]
        store.set("weights_info", pickle.dumps(weights_info))
    weights_info = pickle.loads(store.get("weights_info"))
    for w in (trainer, logprob):
        if w is not None and w is not trainer:
            w.set_trainer_weights_info(weights_info)
    if trainer is not None and rank != T[0]:
        trainer.set_trainer_weights_info(weights_info)

    def sync_all() -> float:
        """The reference's sync_all_weights (orchestrator.py:587-640): every worker runs its own loop."""
        mail.barrier(f"sync{sync_all.n}", n)
        torch.cuda.synchronize()
        t0 = time.time()
        first = True
        for w in (trainer, logprob):
            if w is None:
                continue
            if first:
                group.begin_primary(keep_stash=(is_t + is_l + is_r) > 1)
            else:
                group.begin_secondary()
            asyncio.run(w.sync_weights("sync_group", 0))
            first = False
        if rollout is not None:
            if first:
                group.begin_primary(False)
            else:
                group.begin_secondary()
            rollout.receive_weights(weights_info, group)
        group.end()
        torch.cuda.synchronize()
        mail.barrier(f"sync{sync_all.n}e", n)
        sync_all.n += 1
        return (time.time() - t0) * 1000.0

    sync_all.n = 0
    set_phase("initial weight sync")
    sync_all()  # initial sync, as the reference does at the end of its init (orchestrator.py:545)

    total_steps = args.warmup + args.steps
    rows = synthetic_rows(prompts_per_step * total_steps, arch["vocab_size"], args.prompt_min, args.prompt_max, 0, spq,
                          (args.gen_min, args.gen_max), 0.3)
    batcher = LogprobBatcher(logprob, cfg.max_tokens_per_gpu) if logprob is not None else None
    stats = {"gen_tokens": 0, "samples": 0, "sync_ms": [], "h2d": 0, "d2h": 0, "gen_s": 0.0, "train_s": 0.0}

    def one_step(step: int) -> None:
        set_phase(f"macro-batch {step}")
        step_rows = rows[step * prompts_per_step:(step + 1) * prompts_per_step]
        # 1. generation: prompt i goes to engine i mod r; finished groups go to logprob worker (group mod l)
        if rollout is not None:
            mine = [dict(r) for i, r in enumerate(step_rows) if R[i % len(R)] == rank]
            cnt = [0]

            def on_group(samples):
                mail.post(f"lp/{step}/{L[cnt[0] % len(L)]}", samples)
                cnt[0] += 1

            if len(L) > 1:
                raise RuntimeError("this harness routes every group of an engine round-robin; set one logprob rank per engine")
            tok, dur = rollout.generate(mine, on_group)
            mail.post(f"gen/{step}", (tok, dur))
        # 2. old-policy logprobs
        if logprob is not None:
            expect = len(step_rows)  # one logprob rank: every group arrives here
            got = 0
            box = f"lp/{step}/{rank}"

            def poll() -> bool:
                nonlocal got
                took = False
                while got < expect and mail.ready(box):
                    batcher.queue.extend(mail.take(box))
                    got += 1
                    took = True
                return took

            while got < expect or batcher.queue:
                if not batcher.queue:
                    batcher.queue.extend(mail.take(box))
                    got += 1
                poll()
                done = batcher.run_ready(got < expect, poll)
                if done:
                    mail.post(f"ready/{step}", done)
            mail.post(f"ready/{step}", None)
        # 3. planner on rank 0
        if rank == 0:
            ready: List[dict] = []
            ends = 0
            while ends < len(L):
                got_ = mail.take(f"ready/{step}")
                if got_ is None:
                    ends += 1
                else:
                    ready.extend(got_)
            msgs = plan_microbatches(ready, len(T), cfg.max_tokens_per_gpu, minibatch)
            for ti, r in enumerate(T):
                mail.post(f"train/{step}/{r}", msgs[ti])
            stats["samples"] += len(ready)
            for _ in R:
                tok, dur = mail.take(f"gen/{step}")
                stats["gen_tokens"] += tok
                stats["gen_s"] = max(stats["gen_s"], dur)
        # 4. training
        if trainer is not None:
            t0 = time.time()
            loss = 0.0
            for kind, data in mail.take(f"train/{step}/{rank}"):
                if kind == "microbatch":
                    total = data[0].get("total_non_masked_output_tokens", 0) if data else 0
                    m = trainer.compute_gradients(data, total)
                    loss = float(m.get("loss", 0.0))  # the step's result, read back on the host
                    tk = sum(len(s.get("sample_ids", [])) for s in data)
                    stats["h2d"] += tk * (3 * 8 + 4 * 4)
                    stats["d2h"] += 64
                elif kind == "gradient_step":
                    trainer.apply_gradients()
            stats["train_s"] += time.time() - t0
            stats["last_loss"] = loss
        # 5. weight sync after the optimizer step
        stats["sync_ms"].append(sync_all())

    for s in range(args.warmup):
        one_step(s)
    for k in ("gen_tokens", "samples", "h2d", "d2h"):
        stats[k] = 0
    stats["sync_ms"] = []
    mail.barrier("timed_begin", n)
    torch.cuda.synchronize()
    sampler = ClockSampler()
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t0 = time.time()
    for s in range(args.warmup, total_steps):
        one_step(s)
    ev1.record()
    torch.cuda.synchronize()
    mail.barrier("timed_end", n)
    wall = time.time() - t0
    dev_ms = ev0.elapsed_time(ev1)
    store.set(f"ms/{rank}", pickle.dumps((dev_ms, stats["h2d"] + (batcher.h2d if batcher else 0),
                                          stats["d2h"] + (batcher.d2h if batcher else 0))))
    if rank != 0:
        mail.barrier("exit", n)
        return None
    clocks = sampler.stop()
    per = [pickle.loads(store.get(f"ms/{r}")) for r in range(n)]
    mail.barrier("exit", n)
    dev_s = max(p[0] for p in per) / 1000.0
    samples = stats["samples"]
    par = f"trainer{len(T)}+logprob{len(L)}+rollout{len(R)}" + (" colocated" if n < 3 else "")
    return {
        "impl": "reference", "metric": "GRPO samples/sec (gen tokens/sec and weight-sync ms in extra)",
        "value": samples / dev_s, "unit": "samples/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_s * 1000.0 / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random-init weights, random-token prompts, forced generation lengths)",
        "same_config": True,
        "config": {"model": f"{args.model} architecture", "global_batch": minibatch, "prompts_per_step": prompts_per_step,
                   "samples_per_prompt": spq,
                   "seq_len": f"prompt U[{args.prompt_min},{args.prompt_max}] + generation logU[{args.gen_min},{args.gen_max}]",
                   "parallelism": par, "max_tokens_per_microbatch": cfg.max_tokens_per_gpu, "engine_preset": cfg.vllm_engine_preset,
                   "max_num_seqs": cfg.max_num_seqs, "loss_chunksize": cfg.loss_chunksize,
                   "l2": "working set (weights, KV cache, activations) far larger than the 126 MB L2; no flush needed"},
        "clocks": clocks,
        "e2e": {"value": samples / wall, "unit": "samples/s", "h2d_bytes_per_step": sum(p[1] for p in per) / args.steps,
                "d2h_bytes_per_step": sum(p[2] for p in per) / args.steps,
                "note": "host wall clock around the same macro-batches; the reference builds its tensors from Python lists on the "
                        "host (pageable memory) and reads logprobs and the loss back per batch"},
        "gpu_launches": 0,
        "restated": RESTATED, "stand_ins": sorted(shims),
        "extra": {"gen_tokens_per_s": stats["gen_tokens"] / dev_s, "weight_sync_ms_mean": sum(stats["sync_ms"]) / max(1, len(stats["sync_ms"])),
                  "samples": samples, "gen_tokens": stats["gen_tokens"], "engine_steps": rollout.engine_steps if rollout else None,
                  "sync_broadcasts": group.calls, "last_loss": stats.get("last_loss"),
                  "vllm": "0.22 in-process engine (uniproc executor); reference engine args otherwise"},
    }
