"""Peer-memory collectives on 2+ GPUs against torch.distributed (NCCL) results.

Runs as child processes, one per GPU, with NVLS disabled in NCCL and plain peer loads / stores in our kernels.
Data movement (weight push) must be bit-exact; reductions are compared with a tolerance. The last case lets a
barrier run out on purpose by having one rank skip it: the waiting rank's kernel must return an error status within
its budget while the context stays usable (no fault, no hang)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    # this worker ends with a failure-detection case: NVLS off in NCCL and plain peer loads in our own kernels
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0", "AGRPO_MULTICAST": "0"})
    import torch.distributed as dist

    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.ops import native
    from async_grpo_nccl_b200.parallel import symm

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    trainer_group = dist.new_group(list(range(world)) if world == 2 else list(range(world - 1)))
    try:
        C = native()
        cfg = PRESETS["tiny128"]
        # trainers = every rank but the last when there are more than two GPUs (exercises the sub-group indexing)
        trainers = list(range(world)) if world == 2 else list(range(world - 1))
        layout = ParamLayout(cfg, shard_world=len(trainers))
        plane = symm.SymmetricPlane(dev, layout, C, trainer_ranks=trainers, infer_ranks=list(range(world)))
        comm = plane.trainer_comm()
        ws = plane.weight_sync()
        if comm is None:  # pure inference rank: takes part in the weight push only
            ws.push(None, None)
            torch.cuda.synchronize()
            ws.pg.check()
            full = torch.empty(layout.total, dtype=torch.bfloat16, device=dev)
            dist.broadcast(full, src=0)
            assert torch.equal(ws.buffer, full), "pushed weights differ on the inference rank"
            dist.barrier()
            x = torch.ones(4, device=dev)
            dist.all_reduce(x)
            q.put((rank, "ok"))
            return
        tgroup_world = len(trainers)
        # ---- reduce-scatter + norm ----
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        comm.grad_buffer.copy_(torch.randn(layout.total, device=dev, generator=g))
        full = comm.grad_buffer.clone()
        tg = trainer_group
        dist.all_reduce(full, group=tg)
        shard = torch.zeros(layout.shard_numel(), device=dev)
        comm.reduce_scatter(shard)
        torch.cuda.synchronize()
        comm.pg.check()
        want = torch.cat([full[gs:gs + ln] for lo, gs, ln in layout.local_to_global_ranges(rank)])
        assert torch.allclose(shard, want, rtol=1e-5, atol=1e-5), "reduce-scatter mismatch"
        norm_sq = comm.norm_partials.sum().item()
        assert abs(norm_sq - full.double().pow(2).sum().item()) / full.double().pow(2).sum().item() < 1e-4
        assert float(comm.grad_buffer.abs().max()) == 0.0  # zeroed for the next accumulation
        # ---- AdamW + publish: every rank's parameter buffer equals the gathered bf16 shards ----
        master = torch.cat([torch.full((ln,), float(rank + 1), device=dev) for lo, gs, ln in layout.local_to_global_ranges(rank)])
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        comm.adamw_and_publish(master, m, v, shard.clone(), 1e-2, 0.9, 0.999, 1e-8, 0.0, 1, 1.0)
        torch.cuda.synchronize()
        comm.pg.check()
        gathered = [torch.empty_like(master) for _ in range(tgroup_world)]
        dist.all_gather(gathered, master, group=tg)
        ref = torch.zeros(layout.total, device=dev)
        for r in range(tgroup_world):
            for lo, gs, ln in layout.local_to_global_ranges(r):
                ref[gs:gs + ln] = gathered[r][lo:lo + ln]
        assert torch.equal(comm.param_buffer, ref.to(torch.bfloat16)), "published parameters differ"
        # first Adam step moves by lr * sign(g) (clip coefficient applied to g only changes magnitude of g)
        moved = (master - (rank + 1)).abs()
        assert ((moved - 1e-2).abs() < 1e-4).float().mean().item() > 0.98  # near-zero gradients move less
        # ---- weight push to inference buffers: bit-exact ----
        ws.push(comm.param_buffer, comm.rank)
        torch.cuda.synchronize()
        ws.pg.check()
        assert torch.equal(ws.buffer, comm.param_buffer), "pushed weights differ"
        if world > 2:
            dist.broadcast(comm.param_buffer.clone() if rank == 0 else torch.empty(layout.total, dtype=torch.bfloat16, device=dev), src=0)
        # ---- a barrier partner that never arrives: bounded wait -> error status, context still usable ----
        dist.barrier()
        symm_budget = symm.WAIT_BUDGET_S
        symm.WAIT_BUDGET_S = 0.3
        pg = symm.PeerGroup(plane.flags, list(range(world)), rank, dev, C, slot_base=100)
        if rank == 0:
            pg.barrier()  # rank 1 does not join this one
            torch.cuda.synchronize()
            try:
                pg.check()
                raised = False
            except RuntimeError:
                raised = True
            assert raised, "the lone rank's barrier must report a timeout"
        symm.WAIT_BUDGET_S = symm_budget
        x = torch.ones(4, device=dev)
        dist.all_reduce(x)
        assert x[0].item() == world  # the context and the communicator still work
        q.put((rank, "ok"))
    except Exception as e:  # report instead of leaving the parent waiting
        import traceback

        q.put((rank, f"FAILED: {e!r}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_peer_memory_collectives_match_nccl():
    import torch.multiprocessing as mp

    world = min(8, torch.cuda.device_count())
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29733, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def _worker_sharded(rank, world, port, q):
    """Fully sharded trainer (ag_gemm / gemm_rs over real peer memory) against the resident-parameter trainer: same
    microbatches, two optimizer steps, then the weight push from the slices."""
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    import numpy as np
    import torch.distributed as dist

    from async_grpo_nccl_b200.config import make_config
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.ops import native
    from async_grpo_nccl_b200.packing import pack_for_logprob
    from async_grpo_nccl_b200.parallel import symm
    from async_grpo_nccl_b200.roles.trainer import TrainerCore

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        C = native()
        mcfg = PRESETS["tiny128"]
        cfg = make_config({"model_name_or_path": "tiny128", "train_minibatch_sample_size": 12 * world, "learning_rate": 1e-3,
                           "global_num_verifiers": 0, "max_grad_norm": 1.0})
        ranks = list(range(world))
        layout = ParamLayout(mcfg, shard_world=world)
        plane_ref = symm.SymmetricPlane(dev, layout, C, trainer_ranks=ranks, infer_ranks=ranks)
        plane_z3 = symm.SymmetricPlane(dev, layout, C, trainer_ranks=ranks, infer_ranks=ranks, zero3=True)
        flat = torch.empty(layout.total)
        layout.init_random_(flat, 0)
        flat = flat.to(torch.bfloat16).float()
        ref = TrainerCore(cfg, mcfg, dev, rank, world, None, flat.clone(), comm=plane_ref.trainer_comm())
        z3 = TrainerCore(cfg, mcfg, dev, rank, world, None, flat.clone(), comm=plane_z3.trainer_comm())
        assert z3.zero3 and z3.params is None
        rng = np.random.default_rng(10 + rank)

        def samples(n):
            out = []
            for _ in range(n):
                li, lo = int(rng.integers(4, 40)), int(rng.integers(100, 300))
                L = li + lo
                out.append(dict(sample_ids=rng.integers(0, mcfg.vocab_size, L).astype(np.int32), input_len=li, output_len=lo,
                                advantage=float(rng.normal()), sample_logprobs=np.zeros(L, np.float32),
                                sample_entropies=np.zeros(L, np.float32), reward=1.0))
            return out

        for step in range(2):
            mb = samples(12)
            pb = pack_for_logprob(mb, pin=False).to_device(dev)
            lp, ent = ref.decoder.logprobs(pb, 1.0)
            lp, ent, off = lp.cpu().numpy(), ent.cpu().numpy(), 0
            for s in mb:
                L = len(s["sample_ids"])
                s["sample_logprobs"], s["sample_entropies"] = lp[off:off + L].copy(), ent[off:off + L].copy()
                off += L
            ref.compute_gradients(mb)
            z3.compute_gradients(mb)
            sr, sz = ref.apply_gradients(), z3.apply_gradients()
            assert abs(sr["grad_norm"] - sz["grad_norm"]) < 1e-3 * sr["grad_norm"], (sr["grad_norm"], sz["grad_norm"])
            assert abs(sr["loss"] - sz["loss"]) < 1e-4 * max(1.0, abs(sr["loss"]))
            # the same slice of the fp32 master on both paths. Adam's early steps move by about lr * sign(g), so an
            # element whose gradient is at the noise level of the summation order may go the other way: compare most
            diff = (ref.master - z3.master).abs()
            assert (diff < 1e-5).float().mean().item() > 0.97, (diff < 1e-5).float().mean().item()
        assert z3.comm.weights.gathers_fused > 0
        # gathered slices equal the resident copy of the reference path wherever the masters agree bit for bit
        full = torch.empty(layout.total, dtype=torch.bfloat16, device=dev)
        z3.comm.weights.gather_full(full)
        torch.cuda.synchronize()
        same = ((full.float() - ref.params.float()).abs() < 1e-4).float().mean().item()
        assert same > 0.97, same
        # weight push straight from the slices
        ws = plane_z3.weight_sync()
        src, sharded = z3.sync_source()
        ws.push(src, rank, sharded_src=sharded)
        torch.cuda.synchronize()
        ws.pg.check()
        assert torch.equal(ws.buffer, full), "weights pushed from slices differ from the gathered parameters"
        z3.decoder.check_status()
        z3.comm.pg.check()
        q.put((rank, "ok"))
    except Exception as e:
        import traceback

        q.put((rank, f"FAILED: {e!r}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fully_sharded_trainer_matches_resident_trainer(world):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_sharded, args=(r, world, 29741 + world, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def _worker_multicast(rank, world, port, q):
    """NVSwitch multicast variants (multimem.st push, multimem.ld_reduce reduce-scatter) against plain tensors. Not a
    failure test: every rank stays to the end."""
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port)})
    import torch.distributed as dist

    from async_grpo_nccl_b200.ops import native
    from async_grpo_nccl_b200.parallel import symm

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        C = native()
        n = 1 << 22
        flags = symm.alloc_symmetric(128, torch.int64, dev, dist.group.WORLD)
        wbuf = symm.alloc_symmetric(n, torch.bfloat16, dev, dist.group.WORLD)
        gbuf = symm.alloc_symmetric(n, torch.float32, dev, dist.group.WORLD)
        if not wbuf.mc_ptr or not gbuf.mc_ptr:
            q.put((rank, "skip: no multicast address on this fabric"))
            return
        pg = symm.PeerGroup(flags, list(range(world)), rank, dev, C)
        # push: rank r owns the r-th slice and writes it once through the multicast address
        per = n // world
        src = torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(7)).to(torch.bfloat16)  # same on all ranks
        pg.barrier()
        C.weight_push_mc(src, rank * per, rank * per, per, wbuf.mc_ptr)
        pg.barrier()
        torch.cuda.synchronize()
        pg.check()
        assert torch.equal(wbuf.local, src), "multicast push is not bit-exact"
        # in-switch reduction of every rank's gradient buffer
        g = torch.randn(n, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank))
        gbuf.local.copy_(g)
        total = g.clone()
        dist.all_reduce(total)
        pg.barrier()
        out = torch.zeros(per, device=dev)
        nsq = torch.zeros(1, device=dev)
        C.rs_pull_sumsq_mc(gbuf.mc_ptr, rank * per, 0, per, out, nsq)
        pg.barrier()
        torch.cuda.synchronize()
        pg.check()
        want = total[rank * per:(rank + 1) * per]
        assert torch.allclose(out, want, rtol=1e-5, atol=1e-5), "in-switch reduce-scatter mismatch"
        assert abs(nsq.item() - want.double().pow(2).sum().item()) < 1e-3 * want.double().pow(2).sum().item()
        q.put((rank, "ok"))
    except Exception as e:
        import traceback

        q.put((rank, f"FAILED: {e!r}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_multicast_push_and_in_switch_reduce():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_multicast, args=(r, world, 29751, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    if all(msg.startswith("skip") for _, msg in results):
        pytest.skip(results[0][1])
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


def _worker_tp_engine(rank, world, port, q):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0", "AGRPO_MULTICAST": "0"})
    import numpy as np
    import torch.distributed as dist

    from async_grpo_nccl_b200.engine.engine import RolloutEngine
    from async_grpo_nccl_b200.models.config import ModelConfig
    from async_grpo_nccl_b200.models.decoder import NativeDecoder
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.ops import native
    from async_grpo_nccl_b200.packing import pack_samples
    from async_grpo_nccl_b200.parallel import symm

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        C = native()
        # per-rank shares stay within what the split-K decode GEMMs serve (K >= 512): 4 of 8 heads, 1 of 2 kv heads
        cfg = ModelConfig(vocab_size=2048, hidden_size=1024, intermediate_size=2816, num_hidden_layers=2, num_attention_heads=8,
                          num_key_value_heads=2, head_dim=128, rope_theta=1e4, max_position_embeddings=4096,
                          tie_word_embeddings=True, eos_token_id=1, attention_bias=True)
        layout = ParamLayout(cfg)
        p32 = torch.empty(layout.total)
        layout.init_random_(p32, 0)
        gen = torch.Generator().manual_seed(11)
        for i in range(cfg.num_hidden_layers):  # non-zero biases, so a wrong bias slice shows
            layout.view(p32, f"layers.{i}.bqkv").normal_(0.0, 0.02, generator=gen)
        p16 = (p32 * 2.0).to(torch.bfloat16).to(dev)
        tp = symm.TensorParallelComm(list(range(world)), rank, 64, cfg.hidden_size, dev, C)
        rng = np.random.default_rng(5)
        prompts = [rng.integers(2, cfg.vocab_size, int(rng.integers(4, 30))).astype(np.int32) for _ in range(20)]
        eng = RolloutEngine(cfg, layout, p16, max_seqs=64, max_model_len=128, num_blocks=600, use_cuda_graph=True, tp=tp)
        assert eng.tp_size == world and eng.cache.shape[3] == cfg.num_key_value_heads // world
        for i, pr in enumerate(prompts):
            eng.add_request(i, pr, n=2, max_new_tokens=12, temperature=0.0 if i % 2 == 0 else 1.0, seed=i, ignore_eos=True)
        outs = sorted(eng.run_until_done(), key=lambda o: (o.request_id, o.child))
        torch.cuda.synchronize()
        eng.check_status()
        assert len(outs) == 40
        # every member of the replica produced the same tokens (sampling is replicated, sums are in rank order)
        mine = torch.tensor(np.concatenate([o.output_ids for o in outs]).astype(np.int64), device=dev)
        both = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        assert all(torch.equal(both[0], b) for b in both), "tensor-parallel members disagree on the sampled tokens"
        # greedy tokens are the argmax (up to bf16 noise) of the teacher-forced logits of the unsharded model
        nat = NativeDecoder(cfg, layout, p16)
        wl = layout.view(p16.float(), layout.lm_head_name())
        checked = 0
        for o in outs:
            if o.request_id % 2:
                continue
            pr = prompts[o.request_id]
            full = np.concatenate([pr, o.output_ids])
            pb = pack_samples([{"sample_ids": full, "input_len": len(pr), "output_len": len(o.output_ids)}], pin=False).to_device(dev)
            with torch.no_grad():
                hn, _, _ = nat.hidden(pb)
                z = hn.float() @ wl.t()
            for j, tok in enumerate(o.output_ids):
                row = z[len(pr) - 1 + j]
                top = row.max().item()
                assert row[int(tok)].item() >= top - (0.03 * abs(top) + 0.05), (o.request_id, j)
                checked += 1
        assert checked == 20 * 12
        q.put((rank, "ok"))
    except Exception as e:
        import traceback

        q.put((rank, f"FAILED: {e!r}\n{traceback.format_exc()}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tensor_parallel_engine_matches_unsharded_model():
    """Two SPMD engine ranks with half of the heads / MLP columns each and all-reduce over peer memory: identical tokens on
    both ranks, and greedy tokens that the unsharded model's teacher-forced logits confirm."""
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_tp_engine, args=(r, world, 29771, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, msg in results:
        assert msg == "ok", f"rank {rank}: {msg}"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.timeout(900)
def test_runtime_with_a_tensor_parallel_rollout_replica(tmp_path):
    """The whole role graph on 2 GPUs with generation_tp_size = 2: rank 0 hosts trainer, logprob and the replica's leader,
    rank 1 the follower that replays the leader's engine calls. Two macro-batches with a weight push after each (the
    follower pauses and resumes with the leader) and the weight-sync checksum verified on every rank."""
    from async_grpo_nccl_b200.data import synthetic_prompt_rows
    from async_grpo_nccl_b200.launch import spawn

    arch = dict(vocab_size=2048, hidden_size=1024, intermediate_size=2816, num_hidden_layers=2, num_attention_heads=8,
                num_key_value_heads=2, head_dim=128, rope_theta=1e4, max_position_embeddings=4096, tie_word_embeddings=True,
                eos_token_id=1, attention_bias=True)
    cfg = dict(model_name_or_path="tiny128", model_config=arch, batch_size=4, samples_per_question=4, num_epochs=1,
               train_minibatch_sample_size=8, max_generation_tokens=24, max_tokens_per_gpu=2048, reward_fns=["token_match"],
               global_num_verifiers=0, num_training_gpu_workers=1, num_logprob_gpu_workers=1, num_generation_gpu_workers=2,
               generation_tp_size=2, max_num_seqs=64, vllm_engine_preset="throughput",
               placement={"trainer": [0], "logprob": [0], "rollout": [0, 1]}, learning_rate=1e-4, output_dir=str(tmp_path),
               min_samples_per_checkpoint=10 ** 9, eval_at_start=False, verify_weight_sync_during_init=True)
    rows = synthetic_prompt_rows(8, 2048, 16, 32, seed=0)
    out = spawn(cfg, rows, world=2, max_macro_batches=2, port=29861, timeout_s=300)
    assert out["global_step"] == 2 and out["total_samples_seen"] == 32
    import numpy as np

    assert np.isfinite(out["last"]["training/avg_loss"])
