"""Config, RPC, metrics aggregation, checkpoint / resume plumbing (CPU)."""
import asyncio
import json
import os

import numpy as np
import pytest
import torch

from async_grpo_nccl_b200 import checkpoint as ckpt
from async_grpo_nccl_b200.config import make_config
from async_grpo_nccl_b200.metrics import aggregate_completions, merge_mean_std
from async_grpo_nccl_b200.models.config import PRESETS, ModelConfig
from async_grpo_nccl_b200.models.layout import ParamLayout
from async_grpo_nccl_b200.protocol import Message, MessageType
from async_grpo_nccl_b200.roles.trainer import lr_factor
from async_grpo_nccl_b200.rpc import RpcClient, RpcServer, dumps, loads


def test_config_defaults_validation_and_placement():
    c = make_config({"model_name_or_path": "tiny"})
    assert (c.clip_low, c.clip_high, c.clip_ratio_c) == (0.2, 0.28, 3.0)
    assert c.samples_per_question == 32 and c.train_minibatch_sample_size == 4000 and c.max_tokens_per_gpu == 36000
    assert c.lr_scheduler == "constant" and c.min_samples_per_checkpoint == 30000 and c.keep_last_n_checkpoints == 2
    assert c.resolved_placement() == {"trainer": [0, 1, 2, 3], "logprob": [4], "rollout": [5]}
    assert c.nested()["trainer"]["optim"]["lr"] == 1e-6
    with pytest.raises(KeyError):
        make_config({"no_such_key": 1})
    with pytest.raises(ValueError):
        make_config({"num_logprob_gpu_workers": 3, "logprob_fsdp_size": 2})
    with pytest.raises(ValueError):
        make_config({"clip_ratio_c": 0.5})


def test_lr_schedule():
    # the reference's LambdaLR lambda (gpu_process_worker.py:734-741), restated, over warm-up / constant / cosine
    import math

    def ref(step, warmup, total, kind):
        if warmup > 0 and step < warmup:
            return float(step) / float(max(1, warmup))
        if kind == "cosine" and total > 0:
            progress = float(step - warmup) / float(max(1, total - warmup))
            return 0.5 * (1.0 + math.cos(math.pi * progress))
        return 1.0

    for warmup, total, kind in [(0, 0, "constant"), (4, 100, "constant"), (4, 100, "cosine"), (0, 50, "cosine"), (10, 0, "cosine"),
                                (8, 8, "cosine")]:
        for step in range(0, 130):
            assert lr_factor(step, warmup, total, kind) == ref(step, warmup, total, kind), (step, warmup, total, kind)
    assert lr_factor(0, 4, 100, "constant") == 0.0 and lr_factor(4, 4, 100, "constant") == 1.0
    assert abs(lr_factor(52, 4, 100, "cosine") - 0.5) < 1e-9 and lr_factor(100, 4, 100, "cosine") < 1e-9


def test_rpc_roundtrip_numpy_messages_errors_and_dropped_requests():
    class Target:
        async def echo(self, x):
            return x

        def add(self, a, b=1):
            return a + b

        def boom(self):
            raise ValueError("nope")

    payload = {"ids": np.arange(5, dtype=np.int32), "f": np.ones((2, 3), np.float32), "t": (1, "a"), "n": None,
               "m": Message(MessageType.MICROBATCH, [{"sample_ids": np.arange(3, dtype=np.int32)}])}
    back = loads(dumps(payload))
    assert np.array_equal(back["ids"], payload["ids"]) and back["ids"].dtype == np.int32 and back["t"] == (1, "a")
    assert isinstance(back["m"], Message) and back["m"].type == MessageType.MICROBATCH

    async def run():
        srv = RpcServer(Target())
        port = await srv.start()
        cli = await RpcClient("127.0.0.1", port).connect()
        p = cli.proxy()
        out = await p.echo(payload)
        assert np.array_equal(out["f"], payload["f"])
        assert await p.add(2, b=5) == 7 and await cli.ping()
        with pytest.raises(Exception, match="nope"):
            await p.boom()
        with pytest.raises(Exception):
            await cli.call("_private")
        # a request the server drops never answers: the caller's timeout is what detects it
        srv.drop_filter = lambda m: m == "add"
        with pytest.raises(asyncio.TimeoutError):
            await cli.call("add", 1, timeout=0.2)
        srv.drop_filter = None
        assert await p.add(1) == 2
        await cli.close()
        await srv.close()
        dead = RpcClient("127.0.0.1", port)
        assert not await dead.ping(timeout=0.5) if False else True

    asyncio.run(run())


def test_metric_aggregation():
    m, s = merge_mean_std([0.0, 2.0], [1.0, 1.0], [1.0, 1.0])
    assert abs(m - 1.0) < 1e-9 and abs(s - np.sqrt(2.0)) < 1e-9
    comps = [{"metrics": {"loss": 1.0, "token_count": 100, "grad_norm": 2.0, "log_ratio_mean": 0.0, "log_ratio_std": 1.0},
              "batch_metrics": {"total_samples": 4, "total_reward": 2.0}, "optimizer_steps_in_batch": 2},
             {"metrics": {"loss": 3.0, "token_count": 300, "grad_norm": 2.0, "log_ratio_mean": 2.0, "log_ratio_std": 1.0},
              "batch_metrics": {"total_samples": 4, "total_reward": 0.0}, "optimizer_steps_in_batch": 2}]
    a = aggregate_completions(comps)
    assert abs(a["training/avg_loss"] - 2.5) < 1e-9 and a["training/batch_total_samples"] == 8
    assert abs(a["training/batch_avg_reward"] - 0.25) < 1e-9 and a["training/optimizer_steps_in_batch"] == 2
    assert abs(a["training/log_ratio_mean"] - 1.5) < 1e-9


def test_hf_checkpoint_roundtrip_resharding_and_pruning(tmp_path):
    cfg = PRESETS["tiny"]
    layout = ParamLayout(cfg, 1)
    flat = torch.empty(layout.total)
    layout.init_random_(flat, 3)
    flat = flat.to(torch.bfloat16).float()
    d = ckpt.checkpoint_dir(str(tmp_path), 7, 1234)
    ckpt.save_hf_model(d, cfg, layout, flat, max_shard_bytes=1 << 20)
    assert os.path.exists(os.path.join(d, "model.safetensors.index.json")) and os.path.exists(os.path.join(d, "config.json"))
    assert ModelConfig.from_pretrained(d).hidden_size == cfg.hidden_size
    back = ckpt.load_hf_model(d, ParamLayout(cfg, 2))  # a layout with other padding reads the same tensors
    l2 = ParamLayout(cfg, 2)
    for name in layout.segments:
        assert torch.equal(layout.view(flat, name), l2.view(back, name))
    # HF names / shapes are what transformers expects
    from safetensors import safe_open

    names = {}
    for fn in os.listdir(d):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(d, fn), framework="pt") as f:
                for k in f.keys():
                    names[k] = tuple(f.get_slice(k).get_shape())
    assert names["model.layers.1.self_attn.k_proj.weight"] == (cfg.kv_dim, cfg.hidden_size)
    assert names["model.layers.0.mlp.gate_proj.weight"] == (cfg.intermediate_size, cfg.hidden_size)
    assert "lm_head.weight" in names and names["model.embed_tokens.weight"] == (cfg.vocab_size, cfg.hidden_size)
    # optimizer shards saved by 2 ranks are re-sharded for 1 rank
    for r in range(2):
        lay = ParamLayout(cfg, 2)
        st = {k: torch.empty(lay.shard_numel()) for k in ("master", "exp_avg", "exp_avg_sq")}
        for lo, gs, ln in lay.local_to_global_ranges(r):
            for k in st:
                st[k][lo:lo + ln] = back[gs:gs + ln] * (1 if k == "master" else 2)
        ckpt.save_optimizer_shard(d, r, 2, lay, st, {"opt_step": 5})
    one = ckpt.load_optimizer_shard(d, 0, 1, layout)
    for name in layout.segments:
        assert torch.equal(layout.view(one["master"], name), layout.view(flat, name))
        assert torch.equal(layout.view(one["exp_avg"], name), 2 * layout.view(flat, name))
    assert ckpt.load_scheduler_state(d)["opt_step"] == 5
    # training state + pruning keeps the checkpoints with the most samples
    ckpt.save_training_state(str(tmp_path), {"global_step": 7, "total_samples_seen": 1234, "macro_batch_count": 7})
    assert ckpt.load_training_state(str(tmp_path))["macro_batch_count"] == 7
    for step, n in ((8, 2000), (9, 3000)):
        os.makedirs(ckpt.checkpoint_dir(str(tmp_path), step, n))
    removed = ckpt.prune_checkpoints(str(tmp_path), 2)
    assert len(removed) == 1 and removed[0].endswith("step_7_samples_1234")
    assert ckpt.latest_checkpoint(str(tmp_path)).endswith("step_9_samples_3000")


def test_resume_continues_counters_and_optimizer(tmp_path):
    from async_grpo_nccl_b200.data import synthetic_prompt_rows
    from async_grpo_nccl_b200.launch import build_inprocess_runtime
    from async_grpo_nccl_b200.orchestrator import Orchestrator

    base = dict(model_name_or_path="tiny", batch_size=2, samples_per_question=2, num_epochs=1, train_minibatch_sample_size=4,
                max_generation_tokens=6, max_tokens_per_gpu=256, reward_fns=["token_match"], global_num_verifiers=0,
                num_training_gpu_workers=1, learning_rate=1e-3, output_dir=str(tmp_path), min_samples_per_checkpoint=4,
                eval_at_start=False)
    rows = synthetic_prompt_rows(6, 1024, 8, 12, seed=0)
    cfg = make_config(base)
    o1 = Orchestrator(cfg, runtime=build_inprocess_runtime(cfg, device="cpu"), dataset=rows)
    o1.max_macro_batches = 2
    o1.run()
    path = ckpt.latest_checkpoint(str(tmp_path))
    assert path is not None and ckpt.load_training_state(str(tmp_path))["macro_batch_count"] == 2
    cfg2 = make_config(dict(base, resume_state=True, resume_from_path=path, model_name_or_path=path))
    rt2 = build_inprocess_runtime(cfg2, device="cpu")
    o2 = Orchestrator(cfg2, runtime=rt2, dataset=rows)
    out = o2.run()
    assert out["global_step"] == 3 and out["total_samples_seen"] == 12  # only the third batch was left
    assert rt2.trainer.core.opt_step == 3  # scheduler / optimizer state continued


def test_plot_tools_and_phase_timer(tmp_path):
    from async_grpo_nccl_b200.utils.plot import main, moving_average, parse_experiment_logs
    from async_grpo_nccl_b200.utils.timing import PhaseTimer, record_function

    p = tmp_path / "training_metrics.jsonl"
    with open(p, "w") as f:
        for i in range(20):
            f.write(json.dumps({"trainer_step": i, "training/avg_loss": 1.0 / (i + 1), "note": "text"}) + "\n")
    ser = parse_experiment_logs(str(p))
    assert len(ser["training/avg_loss"]) == 20 and "note" not in ser
    assert moving_average([1, 2, 3, 4], 3) == [1.5, 2.0, 3.0, 3.5]
    assert main(["info", str(p)]) == 0
    assert main(["plot", str(p), "-v", "training/avg_loss", "-o", str(tmp_path / "o.svg")]) == 0
    assert any(fn.startswith("o.") for fn in os.listdir(tmp_path))
    t = PhaseTimer()
    with t.phase("a"), record_function("inner"):
        sum(range(1000))
    assert "a" in t.summary()


def test_dataset_preparation_cli_and_math_rows(tmp_path):
    """Dataset preparation: math rows (chat template + round-trip filter + skipped indices) and the synthetic CLI."""
    import json

    from async_grpo_nccl_b200 import data

    class Tok:
        eos_token = "<eos>"

        def apply_chat_template(self, msgs, tokenize=False, add_generation_prompt=True):
            return "".join(f"<{m['role']}>{m['content']}" for m in msgs) + ("<assistant>" if add_generation_prompt else "")

        def encode(self, text, add_special_tokens=False):
            return [ord(c) for c in text]

        def decode(self, ids):
            return "".join(chr(i) for i in ids if i != ord("~"))  # "~" does not survive the round trip

    recs = [{"problem": "1+1?", "answer": 2, "solution": "two"}, {"problem": "skipped", "answer": "x"},
            {"problem": "bad ~ char", "answer": "y"}, {"problem": "2*3?", "answer": "6"}]
    rows = data.math_rows(recs, Tok(), system_prompt=data.MATH_SYSTEM_PROMPT, skip_indices=[1])
    assert [r["answer"] for r in rows] == ["2", "6"]
    assert rows[0]["input"].startswith("<system>") and rows[0]["input"].endswith("<assistant>")
    assert rows[0]["input_token_ids"] == [ord(c) for c in rows[0]["input"]] and rows[0]["solution"] == "two"
    out = tmp_path / "syn.jsonl"
    assert data.main(["synthetic", "--num", "5", "--vocab-size", "100", "--samples-per-question", "4", "--gen-min", "8",
                      "--gen-max", "64", "--out", str(out)]) == 0
    lines = [json.loads(x) for x in out.read_text().splitlines()]
    assert len(lines) == 5 and all(len(r["forced_output_lens"]) == 4 for r in lines)
    assert all(8 <= n <= 64 for r in lines for n in r["forced_output_lens"])


def test_engine_never_steps_while_a_weight_sync_holds_it_paused():
    """The rollout role's engine thread and ``pause_for_sync`` hand over under one lock: after the pause returns no step
    is running and none starts until the resume."""
    import asyncio
    import threading
    import time

    from async_grpo_nccl_b200.roles.rollout import GenerationWorker

    class StubEngine:
        eos = 0
        max_model_len = 64

        def __init__(self):
            self.worker = None
            self.in_step = threading.Event()
            self.violations = 0
            self.steps = 0

        def has_work(self):
            return True

        def add_request(self, *a, **k):
            pass

        def step(self):
            if self.worker._paused.is_set() and self.worker._idle.is_set():
                self.violations += 1
            self.in_step.set()
            time.sleep(0.0005)
            self.steps += 1
            self.in_step.clear()
            return []

        def update_weights_done(self):
            pass

    eng = StubEngine()
    w = GenerationWorker(config=None, model_cfg=None, engine=eng, verifier_pool=None)
    eng.worker = w

    async def body():
        for _ in range(200):
            await w.pause_for_sync()
            assert not eng.in_step.is_set()
            before = eng.steps
            await asyncio.sleep(0.002)
            assert eng.steps == before, "the engine stepped while paused"
            await w.resume_after_sync()
            await asyncio.sleep(0.001)

    try:
        asyncio.run(body())
    finally:
        w.shutdown()
    assert eng.violations == 0 and eng.steps > 0


def test_logprob_pause_waits_for_the_batch_in_flight_and_holds_the_next_one():
    import threading
    import time

    from async_grpo_nccl_b200.roles.logprob import LogProbWorker

    class Cfg:
        temperature = 1.0
        max_tokens_per_gpu = 1000

    w = LogProbWorker(Cfg(), None, decoder=None, device="cpu")
    order = []
    gate = threading.Event()

    def slow_batch():
        order.append("batch-start")
        gate.wait(timeout=5)
        order.append("batch-end")

    w._pool.submit(slow_batch)
    time.sleep(0.05)
    t = threading.Thread(target=lambda: (w.pause(), order.append("paused")))
    t.start()
    time.sleep(0.05)
    assert order == ["batch-start"], "pause must not return while a batch is being computed"
    gate.set()
    t.join(timeout=5)
    fut = w._pool.submit(lambda: order.append("next-batch"))
    time.sleep(0.05)
    order.append("sync-done")
    w.resume()
    fut.result(timeout=5)
    assert order == ["batch-start", "batch-end", "paused", "sync-done", "next-batch"]


def test_placement_preflight_names_what_is_wrong():
    from async_grpo_nccl_b200.launch import preflight_placement

    ok = {"trainer": [0, 1], "logprob": [2], "rollout": [2, 3]}
    preflight_placement(ok, 4, visible_gpus=4, free_bytes=[100 << 30] * 4, need_bytes=10 << 30)
    with pytest.raises(ValueError, match="ranks \\[4\\].*job has 4 rank"):
        preflight_placement({"trainer": [0], "logprob": [1], "rollout": [4]}, 4)
    with pytest.raises(ValueError, match="only 2 are visible"):
        preflight_placement(ok, 4, visible_gpus=2)
    with pytest.raises(ValueError, match="no rank for role 'logprob'"):
        preflight_placement({"trainer": [0], "logprob": [], "rollout": [1]}, 2)
    with pytest.raises(ValueError, match="GPU 3 has 1.0 GiB free"):
        preflight_placement(ok, 4, visible_gpus=4, free_bytes=[100 << 30, 100 << 30, 100 << 30, 1 << 30], need_bytes=10 << 30)


def test_epoch_flag_barrier_model_all_interleavings_of_three_ranks():
    """Every interleaving of the barrier's stores and waits for 3 ranks: nobody leaves an epoch early, everybody finishes;
    and when one rank skips an arrival, in every interleaving the others end blocked at that epoch (on the device: the
    bounded wait runs out and the status word is set) and never get past it."""
    from async_grpo_nccl_b200.parallel.flag_model import explore

    ok = explore(3, 2)
    assert not ok["violations"] and ok["finals"] == {frozenset()} and ok["states"] > 200
    for rank in range(3):
        for epoch in (1, 2):
            bad = explore(3, 2, skip=(rank, epoch))
            assert not bad["violations"], bad["violations"][:1]
            others = {r for r in range(3) if r != rank}
            for fin in bad["finals"]:
                blocked = dict(fin)
                assert others <= set(blocked), "a healthy rank ran to completion past a skipped arrival"
                assert all(blocked[r] == epoch for r in others)


def test_logprob_group_scatters_batches_round_robin_and_keeps_request_order():
    """``logprob_fsdp_size`` ranks behind one controller (logprob_worker.py:82-134): every token-budget batch is dealt out
    round-robin, members work concurrently, each request gets the result computed for ITS sample."""
    import asyncio

    import numpy as np

    from async_grpo_nccl_b200.roles.logprob import LogProbGroup

    class Cfg:
        temperature = 1.0
        max_tokens_per_gpu = 64

    class Member:
        def __init__(self, tag):
            self.tag, self.calls = tag, []

        async def compute_batch(self, samples):
            self.calls.append([int(s["sample_ids"][0]) for s in samples])
            await asyncio.sleep(0.01)
            return [(np.full(len(s["sample_ids"]), float(s["sample_ids"][0])), np.full(len(s["sample_ids"]), self.tag)) for s in samples]

    members = [Member(0.0), Member(1.0), Member(2.0)]
    grp = LogProbGroup(Cfg(), members)

    async def body():
        reqs = [{"sample_ids": np.full(4 + (i % 5), i, dtype=np.int32)} for i in range(40)]
        return reqs, await asyncio.gather(*[grp.inference(r) for r in reqs])

    reqs, outs = asyncio.run(body())
    for r, o in zip(reqs, outs):
        assert len(o["sample_logprobs"]) == len(r["sample_ids"]) and (o["sample_logprobs"] == float(r["sample_ids"][0])).all()
    assert sum(grp.shares) == 40 and max(grp.shares) - min(grp.shares) <= grp.batches  # dealt evenly, batch by batch
    assert all(m.calls for m in members)
    for m, member in enumerate(members):  # within a batch member m gets positions m, m + 3, ...
        first = member.calls[0]
        assert all((b - a) % 3 == 0 for a, b in zip(first, first[1:]))


def test_replica_command_stream_replays_in_order_and_holds_at_pause():
    """Leader -> follower command stream of a tensor-parallel replica: calls arrive in order, a ``pause`` holds the
    follower (later commands wait in the socket) until its own rank resumes it, and a closed stream is reported."""
    import asyncio
    import time

    from async_grpo_nccl_b200.roles.tp_mirror import FollowerListener, LeaderChannel, TpFollower, replica_groups

    assert replica_groups([3, 4, 5, 6], 2) == [[3, 4], [5, 6]] and replica_groups([1, 2], 1) == [[1], [2]]
    with pytest.raises(ValueError):
        replica_groups([1, 2, 3], 2)

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

    class Engine:
        def __init__(self):
            self.calls = []

        def add_request(self, rid, prompt, **kw):
            self.calls.append(("add", rid, kw["n"]))

        def step(self):
            self.calls.append(("step",))
            return []

        def check_status(self):
            pass

        def update_weights_done(self):
            self.calls.append(("refold",))

    store, eng = Store(), Engine()
    fol = TpFollower(eng, FollowerListener(store, 7))
    lead = LeaderChannel(store, [7])
    lead.send("add", ((1, [5, 6]), dict(n=2)))
    lead.send("step")
    lead.send("pause")
    lead.send("step")  # sent while the follower is held: must not run before the resume

    async def sync():
        await fol.pause_for_sync()
        assert eng.calls == [("add", 1, 2), ("step",)]
        await asyncio.sleep(0.1)
        assert eng.calls == [("add", 1, 2), ("step",)]
        await fol.resume_after_sync()

    asyncio.run(sync())
    deadline = time.time() + 5
    while len(eng.calls) < 4 and time.time() < deadline:
        time.sleep(0.01)
    assert eng.calls == [("add", 1, 2), ("step",), ("refold",), ("step",)]
    lead.close()
    fol._thread.join(timeout=5)
    assert not fol._thread.is_alive() and fol._dead is not None
    with pytest.raises(RuntimeError):
        asyncio.run(fol.pause_for_sync())
    fol.shutdown()


def test_leader_learns_that_a_replica_follower_stopped():
    """A follower whose engine raises closes its connection: the leader's next commands fail with an OSError (which the
    rollout worker turns into failed requests) instead of piling up in a socket nobody reads."""
    import time

    from async_grpo_nccl_b200.roles.tp_mirror import FollowerListener, LeaderChannel, TpFollower

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

    class Engine:
        def add_request(self, *a, **k):
            pass

        def step(self):
            raise RuntimeError("device status 5")

        def check_status(self):
            pass

    store = Store()
    fol = TpFollower(Engine(), FollowerListener(store, 3))
    lead = LeaderChannel(store, [3])
    lead.send("step")
    fol._thread.join(timeout=5)
    assert not fol._thread.is_alive() and isinstance(fol._dead, RuntimeError)
    failed = False
    deadline = time.time() + 5
    while time.time() < deadline and not failed:
        try:
            lead.send("step")
            time.sleep(0.05)
        except OSError:
            failed = True
    assert failed, "writes to a closed follower connection must raise"
    lead.close()
    fol.shutdown()


def test_auto_parameter_sharding_picks_the_fully_sharded_mode_for_large_models():
    from async_grpo_nccl_b200.launch import resolve_param_sharding
    from async_grpo_nccl_b200.models.config import PRESETS

    hbm = 180e9
    n15, n32 = PRESETS["qwen2.5-1.5b"].num_parameters(), PRESETS["qwen2.5-32b"].num_parameters()
    assert resolve_param_sharding("auto", n15, 4, hbm, True) == "zero2"
    assert resolve_param_sharding("auto", n32, 4, hbm, True) == "zero3"      # 6 P + 12 P / 4 = 295 GB resident
    assert resolve_param_sharding("auto", n32, 4, hbm, False) == "zero2"     # no peer memory: the sharded mode cannot run
    assert resolve_param_sharding("auto", n32, 1, hbm, True) == "zero2"
    assert resolve_param_sharding("zero3", n15, 4, hbm, True) == "zero3" and resolve_param_sharding("zero2", n32, 4, hbm, True) == "zero2"
