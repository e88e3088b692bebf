"""The full role graph as separate processes over gloo + RPC on CPU: 2 trainer ranks (sharded optimizer state),
1 rank hosting logprob + rollout. Checks that collectives line up, that both trainer ranks end with the same
parameters and that the weight sync delivered them to the inference rank."""
import numpy as np
import pytest

from async_grpo_nccl_b200.data import synthetic_prompt_rows
from async_grpo_nccl_b200.launch import spawn


@pytest.mark.timeout(600)
def test_three_process_pipeline(tmp_path):
    cfg = dict(model_name_or_path="tiny", batch_size=4, samples_per_question=4, num_epochs=1, train_minibatch_sample_size=8,
               max_generation_tokens=10, max_tokens_per_gpu=200, reward_fns=["token_match"], global_num_verifiers=0,
               num_training_gpu_workers=2, num_logprob_gpu_workers=1, num_generation_gpu_workers=1,
               placement={"trainer": [0, 1], "logprob": [2], "rollout": [2]}, learning_rate=1e-3, output_dir=str(tmp_path),
               min_samples_per_checkpoint=10 ** 9, eval_at_start=False, verify_weight_sync_during_init=True)
    rows = synthetic_prompt_rows(8, 1024, 16, 32, seed=0)
    out = spawn(cfg, rows, world=3, max_macro_batches=2, port=29711, timeout_s=500)
    assert out["global_step"] == 2
    assert out["total_samples_seen"] == 32
    last = out["last"]
    assert last["training/optimizer_steps_in_batch"] == 2
    assert np.isfinite(last["training/avg_loss"]) and last["training/grad_norm"] > 0


def _samples(vocab, n, seed):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n):
        li, lo = int(rng.integers(3, 12)), int(rng.integers(4, 20))
        L = li + lo
        out.append(dict(sample_ids=rng.integers(0, vocab, L).astype(np.int32), input_len=li, output_len=lo,
                        advantage=float(rng.normal()), sample_logprobs=(-rng.random(L) * 3).astype(np.float32),
                        sample_entropies=np.zeros(L, np.float32), reward=float(rng.random() < 0.5)))
    return out


def _sharded_rank(rank, world, port, q):
    import os

    import torch
    import torch.distributed as dist

    from async_grpo_nccl_b200.config import make_config
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.roles.trainer import TrainerCore

    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mcfg = PRESETS["tiny"]
        cfg = make_config({"model_name_or_path": "tiny", "train_minibatch_sample_size": 12, "learning_rate": 1e-3,
                           "global_num_verifiers": 0, "max_grad_norm": 1.0})
        layout = ParamLayout(mcfg, shard_world=world)
        flat = torch.empty(layout.total)
        layout.init_random_(flat, 0)
        core = TrainerCore(cfg, mcfg, torch.device("cpu"), rank, world, dist.group.WORLD, flat.clone())
        # rank 0 holds 8 of the 12 samples, rank 1 the other 4; the second dispatch gives rank 1 a dummy microbatch
        mine = _samples(mcfg.vocab_size, 12, 5)[:8] if rank == 0 else _samples(mcfg.vocab_size, 12, 5)[8:]
        core.compute_gradients(mine[:4])
        core.compute_gradients(mine[4:] if rank == 0 else [{"dummy": True}])
        summary = core.apply_gradients()
        full = core.full_master_fp32()
        if rank == 0:
            q.put(("ok", full.numpy(), summary["grad_norm"], layout.total))
    except Exception as e:  # report instead of leaving the parent waiting
        import traceback

        if rank == 0:
            q.put(("FAILED", f"{e!r}\n{traceback.format_exc()}", 0.0, 0))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_sharded_trainer_ranks_make_the_single_rank_update():
    """Sharded data-parallel semantics (the reference's FSDP2 + loss scaling): two ranks with different microbatches, a
    dummy microbatch on the rank that runs out, reduce-scatter, global-norm clip and AdamW on the shards give the same
    parameters as one rank that sees every sample."""
    import torch
    import torch.multiprocessing as mp

    from async_grpo_nccl_b200.config import make_config
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.roles.trainer import TrainerCore

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_sharded_rank, args=(r, 2, 29723, q)) for r in range(2)]
    for p in procs:
        p.start()
    status, full2, norm2, total2 = q.get(timeout=500)
    for p in procs:
        p.join(timeout=60)
    assert status == "ok", full2
    mcfg = PRESETS["tiny"]
    cfg = make_config({"model_name_or_path": "tiny", "train_minibatch_sample_size": 12, "learning_rate": 1e-3,
                       "global_num_verifiers": 0, "max_grad_norm": 1.0})
    layout1 = ParamLayout(mcfg, shard_world=1)
    flat = torch.empty(layout1.total)
    layout1.init_random_(flat, 0)
    one = TrainerCore(cfg, mcfg, torch.device("cpu"), init_flat_fp32=flat.clone())
    alls = _samples(mcfg.vocab_size, 12, 5)
    for mb in (alls[:4], alls[4:8], alls[8:]):
        one.compute_gradients(mb)
    s1 = one.apply_gradients()
    assert abs(s1["grad_norm"] - norm2) < 1e-4 * max(1.0, s1["grad_norm"])
    # compare parameter by parameter (the two layouts pad their units differently)
    layout2 = ParamLayout(mcfg, shard_world=2)
    assert layout2.total == total2
    f2 = torch.from_numpy(full2)
    for name in layout1.segments:
        a, b = layout1.view(one.master, name), layout2.view(f2, name)
        assert torch.allclose(a, b, rtol=1e-5, atol=2e-6), name


@pytest.mark.timeout(600)
def test_rollout_rank_streams_logprob_requests_to_another_rank(tmp_path):
    """Trainer, logprob and rollout each on a rank of their own: the rollout rank asks the logprob rank for a sample's
    old-policy log-probabilities over RPC as soon as that sample finishes (no hop through rank 0)."""
    cfg = dict(model_name_or_path="tiny", batch_size=4, samples_per_question=4, num_epochs=1, train_minibatch_sample_size=16,
               max_generation_tokens=10, max_tokens_per_gpu=400, reward_fns=["token_match"], global_num_verifiers=0,
               num_training_gpu_workers=1, num_logprob_gpu_workers=1, num_generation_gpu_workers=1,
               placement={"trainer": [0], "logprob": [1], "rollout": [2]}, learning_rate=1e-3, output_dir=str(tmp_path),
               min_samples_per_checkpoint=10 ** 9, eval_at_start=False, stream_logprobs=True)
    rows = synthetic_prompt_rows(8, 1024, 16, 32, seed=0)
    out = spawn(cfg, rows, world=3, max_macro_batches=2, port=29735, timeout_s=500)
    assert out["global_step"] == 2 and out["total_samples_seen"] == 32
    last = out["last"]
    assert last["training/optimizer_steps_in_batch"] == 1
    assert np.isfinite(last["training/avg_loss"]) and last["training/grad_norm"] > 0


def _save_rank(rank, world, port, path, q):
    import os

    import torch
    import torch.distributed as dist

    from async_grpo_nccl_b200 import checkpoint as ckpt
    from async_grpo_nccl_b200.config import make_config
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.roles.trainer import TrainerCore

    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mcfg = PRESETS["tiny"]
        cfg = make_config({"model_name_or_path": "tiny", "train_minibatch_sample_size": 8, "learning_rate": 1e-3,
                           "global_num_verifiers": 0, "lr_warmup_steps": 2})
        layout = ParamLayout(mcfg, shard_world=world)
        flat = torch.empty(layout.total)
        layout.init_random_(flat, 0)
        core = TrainerCore(cfg, mcfg, torch.device("cpu"), rank, world, dist.group.WORLD, flat.clone())
        for step in range(3):
            core.compute_gradients(_samples(mcfg.vocab_size, 8, 10 + step)[rank * 4:(rank + 1) * 4])
            core.apply_gradients()
        ckpt.save_optimizer_shard(path, rank, world, layout, core.optimizer_state(), core.scheduler_state())
        full = core.full_master_fp32()
        if rank == 0:
            q.put(("ok", full.numpy()))
    except Exception as e:
        if rank == 0:
            q.put(("FAILED", repr(e)))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_optimizer_state_written_by_two_ranks_resumes_on_one(tmp_path):
    """Resume with another trainer count: shards saved by 2 ranks are re-cut for 1 rank; master weights, both Adam moments
    and the schedule position come back, the compute copy is rebuilt from the masters, and the next step continues from them."""
    import torch
    import torch.multiprocessing as mp

    from async_grpo_nccl_b200 import checkpoint as ckpt
    from async_grpo_nccl_b200.config import make_config
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.roles.trainer import TrainerCore

    path = str(tmp_path / "ck")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_save_rank, args=(r, 2, 29747, path, q)) for r in range(2)]
    for p in procs:
        p.start()
    status, full2 = q.get(timeout=500)
    for p in procs:
        p.join(timeout=60)
    assert status == "ok", full2
    mcfg = PRESETS["tiny"]
    cfg = make_config({"model_name_or_path": "tiny", "train_minibatch_sample_size": 8, "learning_rate": 5e-4,
                       "global_num_verifiers": 0, "lr_warmup_steps": 2})
    one = TrainerCore(cfg, mcfg, torch.device("cpu"))
    before = one.master.clone()
    assert one.load_optimizer_checkpoint(path)
    assert not torch.equal(before, one.master)
    l1, l2 = one.layout, ParamLayout(mcfg, shard_world=2)
    f2 = torch.from_numpy(full2)
    for name in l1.segments:
        assert torch.equal(l1.view(one.master, name), l2.view(f2, name)), name
        assert torch.equal(l1.view(one.params, name), l1.view(one.master, name).to(one.params.dtype)), name
    assert one.opt_step == 3 and one.exp_avg.abs().sum() > 0 and one.exp_avg_sq.abs().sum() > 0
    assert one.base_lr == 5e-4, "the resumed run's own learning rate applies"
    # moments agree with the shards on disk, segment by segment
    saved = [ckpt.load_optimizer_shard(path, r, 2, l2) for r in range(2)]
    full_m = torch.zeros(l2.total)
    for r in range(2):
        for lo, gs, ln in l2.local_to_global_ranges(r):
            full_m[gs:gs + ln] = saved[r]["exp_avg"][lo:lo + ln]
    for name in l1.segments:
        assert torch.equal(l1.view(one.exp_avg, name), l2.view(full_m, name)), name
    one.compute_gradients(_samples(mcfg.vocab_size, 8, 99))
    s = one.apply_gradients()
    assert s["optimizer_step"] == 4 and s["lr"] == 5e-4
    assert not one.load_optimizer_checkpoint(str(tmp_path / "nothing_here"))


@pytest.mark.timeout(600)
def test_multi_process_runtime_reloads_optimizer_state_on_resume(tmp_path):
    """Run, checkpoint, then start again with ``resume_from_path`` and a different trainer count: the trainer ranks
    reload (and re-shard) the optimizer state inside ``DistributedRuntime`` and the run carries on."""
    from async_grpo_nccl_b200 import checkpoint as ckpt

    base = dict(model_name_or_path="tiny", batch_size=4, samples_per_question=4, num_epochs=1, train_minibatch_sample_size=8,
                max_generation_tokens=8, max_tokens_per_gpu=200, reward_fns=["token_match"], global_num_verifiers=0,
                num_logprob_gpu_workers=1, num_generation_gpu_workers=1, learning_rate=1e-3, output_dir=str(tmp_path),
                eval_at_start=False)
    rows = synthetic_prompt_rows(8, 1024, 16, 32, seed=0)
    first = dict(base, num_training_gpu_workers=2, placement={"trainer": [0, 1], "logprob": [2], "rollout": [2]},
                 min_samples_per_checkpoint=16)
    out = spawn(first, rows, world=3, max_macro_batches=1, port=29759, timeout_s=500)
    assert out["global_step"] == 1
    path = ckpt.latest_checkpoint(str(tmp_path))
    assert path is not None and ckpt.load_scheduler_state(path)["opt_step"] == 2
    second = dict(base, num_training_gpu_workers=1, placement={"trainer": [0], "logprob": [1], "rollout": [1]},
                  min_samples_per_checkpoint=10 ** 9, model_name_or_path=path, model_config="tiny" if False else None,
                  resume_from_path=path, resume_state=True, verify_weight_sync_during_init=True)
    second = {k: v for k, v in second.items() if v is not None}
    out2 = spawn(second, rows, world=2, max_macro_batches=1, port=29771, timeout_s=500)
    assert out2["global_step"] == 2 and np.isfinite(out2["last"]["training/avg_loss"])


@pytest.mark.timeout(600)
def test_two_logprob_ranks_behind_one_controller(tmp_path):
    """``logprob_fsdp_size=2``: two logprob ranks form one service whose token-budget batches are scattered over both."""
    cfg = dict(model_name_or_path="tiny", batch_size=4, samples_per_question=4, num_epochs=1, train_minibatch_sample_size=16,
               max_generation_tokens=10, max_tokens_per_gpu=400, reward_fns=["token_match"], global_num_verifiers=0,
               num_training_gpu_workers=1, num_logprob_gpu_workers=2, logprob_fsdp_size=2, num_generation_gpu_workers=1,
               placement={"trainer": [0], "logprob": [1, 2], "rollout": [3]}, learning_rate=1e-3, output_dir=str(tmp_path),
               min_samples_per_checkpoint=10 ** 9, eval_at_start=False, stream_logprobs=False)
    rows = synthetic_prompt_rows(8, 1024, 16, 32, seed=0)
    out = spawn(cfg, rows, world=4, max_macro_batches=2, port=29795, timeout_s=500)
    assert out["global_step"] == 2 and out["total_samples_seen"] == 32
    assert np.isfinite(out["last"]["training/avg_loss"]) and out["last"]["training/grad_norm"] > 0


@pytest.mark.timeout(600)
def test_replica_of_two_rollout_ranks_follows_its_leader(tmp_path):
    """generation_tp_size=2 on CPU ranks: ranks 1 and 2 form one engine replica. Rank 1 leads (request queue, results,
    verifier); rank 2 replays the leader's engine calls from the command stream and takes part in every weight sync. The
    run must finish with both macro-batches trained and the weight-sync checksums equal on every rank (which also shows
    that the follower paused and resumed with the leader)."""
    cfg = dict(model_name_or_path="tiny", batch_size=4, samples_per_question=4, num_epochs=1, train_minibatch_sample_size=8,
               max_generation_tokens=10, max_tokens_per_gpu=200, reward_fns=["token_match"], global_num_verifiers=0,
               num_training_gpu_workers=1, num_logprob_gpu_workers=1, num_generation_gpu_workers=2, generation_tp_size=2,
               placement={"trainer": [0], "logprob": [0], "rollout": [1, 2]}, learning_rate=1e-3, output_dir=str(tmp_path),
               min_samples_per_checkpoint=10 ** 9, eval_at_start=False, verify_weight_sync_during_init=True)
    rows = synthetic_prompt_rows(8, 1024, 16, 32, seed=0)
    out = spawn(cfg, rows, world=3, max_macro_batches=2, port=29817, timeout_s=500)
    assert out["global_step"] == 2
    assert out["total_samples_seen"] == 32
    assert np.isfinite(out["last"]["training/avg_loss"])


@pytest.mark.timeout(900)
def test_named_eight_rank_placement(tmp_path):
    """The placement of the 8-GPU configuration (4 sharded trainer ranks, 1 logprob rank, 3 rollout ranks) as 8 CPU ranks:
    prompts spread over three engines, streamed logprob requests to one rank, microbatches planned over four trainer
    ranks with dummy batches where a rank has nothing, and the weight push reaching all four inference ranks."""
    cfg = dict(model_name_or_path="tiny", batch_size=6, samples_per_question=4, num_epochs=1, train_minibatch_sample_size=12,
               max_generation_tokens=8, max_tokens_per_gpu=150, reward_fns=["token_match"], global_num_verifiers=0,
               num_training_gpu_workers=4, num_logprob_gpu_workers=1, num_generation_gpu_workers=3,
               placement={"trainer": [0, 1, 2, 3], "logprob": [4], "rollout": [5, 6, 7]}, learning_rate=1e-3,
               output_dir=str(tmp_path), min_samples_per_checkpoint=10 ** 9, eval_at_start=False,
               verify_weight_sync_during_init=True, eager_microbatch_dispatch=True)
    rows = synthetic_prompt_rows(12, 1024, 16, 32, seed=0)
    out = spawn(cfg, rows, world=8, max_macro_batches=2, port=29841, timeout_s=800)
    assert out["global_step"] == 2
    assert out["total_samples_seen"] == 48
    last = out["last"]
    assert last["training/optimizer_steps_in_batch"] == 2
    assert np.isfinite(last["training/avg_loss"]) and last["training/grad_norm"] > 0


@pytest.mark.timeout(900)
def test_launcher_command_line_single_process_and_three_ranks(tmp_path):
    """``python -m async_grpo_nccl_b200.launch --config run.json``: plain (all roles in one process) and under
    ``torch.distributed.run`` with three CPU ranks (rank 0 drives, the others serve)."""
    import json
    import os
    import subprocess
    import sys

    from async_grpo_nccl_b200.data import synthetic_prompt_rows

    rows = synthetic_prompt_rows(8, 1024, 16, 32, seed=0)
    data = tmp_path / "train.jsonl"
    with open(data, "w") as f:
        for r in rows:
            f.write(json.dumps({k: (v.tolist() if hasattr(v, "tolist") else v) for k, v in r.items()}) + "\n")
    cfg = dict(model_name_or_path="tiny", data_path=str(data), batch_size=4, samples_per_question=4, num_epochs=1,
               train_minibatch_sample_size=8, max_generation_tokens=10, max_tokens_per_gpu=200, reward_fns=["token_match"],
               global_num_verifiers=0, num_training_gpu_workers=1, learning_rate=1e-3, output_dir=str(tmp_path / "out1"),
               min_samples_per_checkpoint=10 ** 9, eval_at_start=False)
    path = tmp_path / "run.json"
    path.write_text(json.dumps(cfg))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    one = subprocess.run([sys.executable, "-m", "async_grpo_nccl_b200.launch", "--config", str(path), "--max-macro-batches", "1",
                          "--set", "learning_rate=0.002"], capture_output=True, text=True, env=env, timeout=400)
    assert one.returncode == 0, one.stderr[-2000:]
    out = json.loads(one.stdout.strip().splitlines()[-1])
    assert out["global_step"] == 1 and out["total_samples_seen"] == 16
    three = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "3", "--master-addr",
                            "127.0.0.1", "--master-port", "29873", "-m", "async_grpo_nccl_b200.launch", "--config", str(path),
                            "--max-macro-batches", "1", "--set", f"output_dir={tmp_path / 'out3'}", "--set", "num_training_gpu_workers=2",
                            "--set", 'placement={"trainer": [0, 1], "logprob": [2], "rollout": [2]}'],
                           capture_output=True, text=True, env=env, timeout=600)
    assert three.returncode == 0, three.stderr[-3000:]
    line = [l for l in three.stdout.strip().splitlines() if l.startswith("{")][-1]
    assert json.loads(line)["global_step"] == 1
