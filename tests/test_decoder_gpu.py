"""Native decoder / trainer / engine against the PyTorch oracle on small models."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _samples(cfg, n, rng, lo=10, hi=300):
    out = []
    for _ in range(n):
        li, lo_ = int(rng.integers(4, 40)), int(rng.integers(lo, hi))
        L = li + lo_
        out.append(dict(sample_ids=rng.integers(0, cfg.vocab_size, L).astype(np.int32), input_len=li, output_len=lo_,
                        advantage=float(rng.normal()), sample_logprobs=np.zeros(L, np.float32),
                        sample_entropies=np.zeros(L, np.float32), reward=float(rng.random() < 0.5)))
    return out


@pytest.mark.parametrize("preset", ["tiny128", "tiny"])
def test_forward_backward_matches_oracle(preset):
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.decoder import GradSink, LossConfig, NativeDecoder, OracleDecoder
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.packing import pack_samples

    cfg = PRESETS[preset]
    layout = ParamLayout(cfg)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = p32.to(torch.bfloat16).to(DEV)
    rng = np.random.default_rng(0)
    pb = pack_samples(_samples(cfg, 5, rng), pin=False).to_device(DEV)
    lc = LossConfig(kl_beta=0.0, temperature=1.0)
    pref = p16.float().clone().requires_grad_(True)
    orc = OracleDecoder(cfg, layout, pref)
    with torch.no_grad():
        lp0, ent0 = orc.logprobs(pb, 1.0)
    pb.old_logprobs.copy_(lp0 + 0.02 * torch.randn_like(lp0))  # ratios stay away from the clip boundaries
    loss, stats_ref = orc.loss(pb, lc, 0.5)
    loss.backward()
    for recompute in (False, True):
        nat = NativeDecoder(cfg, layout, p16, recompute=recompute)
        sink = GradSink(layout, DEV)
        stats = nat.forward_backward(pb, lc, 0.5, sink)
        torch.cuda.synchronize()
        nat.check_status()
        lval = stats[1].item() / max(1, stats[0].item()) * 0.5
        assert abs(lval - loss.item()) < 2e-3 * max(1.0, abs(loss.item()))
        assert stats[0].item() == stats_ref[0].item()
        for name in layout.segments:
            a, b = layout.view(sink.flat, name), layout.view(pref.grad, name)
            cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
            assert cos > 0.995, (name, cos)
            assert (a - b).abs().max().item() < 0.06 * b.abs().max().item() + 1e-7, name
    lpn, entn = nat.logprobs(pb, 1.0)
    assert (lpn - lp0).abs().max().item() < 3e-2 and (entn - ent0).abs().max().item() < 3e-2


def test_long_packed_microbatch_with_recompute_matches_oracle():
    """A 32 768-token packed microbatch that holds one 16 384-token sequence next to short ones, through forward_backward
    with per-layer recompute: loss, token count, log-probabilities and every gradient against the fp32 PyTorch oracle."""
    import dataclasses

    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.decoder import GradSink, LossConfig, NativeDecoder, OracleDecoder
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.packing import pack_samples

    cfg = dataclasses.replace(PRESETS["tiny128"], max_position_embeddings=32768)
    layout = ParamLayout(cfg)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = p32.to(torch.bfloat16).to(DEV)
    rng = np.random.default_rng(2)

    def sample(li, lo_):
        L = li + lo_
        return dict(sample_ids=rng.integers(0, cfg.vocab_size, L).astype(np.int32), input_len=li, output_len=lo_,
                    advantage=float(rng.normal()), sample_logprobs=np.zeros(L, np.float32),
                    sample_entropies=np.zeros(L, np.float32), reward=float(rng.random() < 0.5))

    samples = [sample(40, 16384 - 40)]
    total = 16384
    while total < 32768 - 700:
        li, lo_ = int(rng.integers(4, 100)), int(rng.integers(50, 600))
        samples.insert(int(rng.integers(0, len(samples) + 1)), sample(li, lo_))
        total += li + lo_
    samples.append(sample(20, 32768 - total - 20))
    pb = pack_samples(samples, pin=False).to_device(DEV)
    assert pb.T == 32768
    lc = LossConfig(kl_beta=0.0, temperature=1.0)
    pref = p16.float().clone().requires_grad_(True)
    orc = OracleDecoder(cfg, layout, pref)
    with torch.no_grad():
        lp0, _ = orc.logprobs(pb, 1.0)
    pb.old_logprobs.copy_(lp0 + 0.02 * torch.randn_like(lp0))
    loss, stats_ref = orc.loss(pb, lc, 0.5)
    loss.backward()
    nat = NativeDecoder(cfg, layout, p16, recompute=True)
    sink = GradSink(layout, DEV)
    stats = nat.forward_backward(pb, lc, 0.5, sink)
    torch.cuda.synchronize()
    nat.check_status()
    lval = stats[1].item() / max(1, stats[0].item()) * 0.5
    assert abs(lval - loss.item()) < 2e-3 * max(1.0, abs(loss.item()))
    assert stats[0].item() == stats_ref[0].item()
    for name in layout.segments:
        a, b = layout.view(sink.flat, name), layout.view(pref.grad, name)
        cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
        assert cos > 0.99, (name, cos)
    lpn, _ = nat.logprobs(pb, 1.0)
    assert (lpn - lp0).abs().max().item() < 4e-2


def test_trainer_step_matches_oracle_step():
    """One full optimizer step (two microbatches, clip, AdamW) on the GPU kernels equals the oracle trainer on CPU."""
    from async_grpo_nccl_b200.config import make_config
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.roles.trainer import TrainerCore

    mcfg = PRESETS["tiny128"]
    cfg = make_config({"model_name_or_path": "tiny128", "train_minibatch_sample_size": 8, "learning_rate": 1e-3,
                       "global_num_verifiers": 0, "max_grad_norm": 1.0})
    rng = np.random.default_rng(1)
    mb1, mb2 = _samples(mcfg, 4, rng, 10, 120), _samples(mcfg, 4, rng, 10, 120)
    from async_grpo_nccl_b200.models.layout import ParamLayout

    layout = ParamLayout(mcfg)
    flat = torch.empty(layout.total)
    layout.init_random_(flat, 0)
    flat = flat.to(torch.bfloat16).float()  # both sides start from bf16-representable weights
    gpu = TrainerCore(cfg, mcfg, torch.device(DEV), init_flat_fp32=flat.clone())
    cpu = TrainerCore(cfg, mcfg, torch.device("cpu"), init_flat_fp32=flat.clone())
    # old logprobs = current policy's, so every ratio is 1 and no token sits on a clip boundary
    for core in (gpu, cpu):
        pass
    from async_grpo_nccl_b200.packing import pack_for_logprob

    for mb in (mb1, mb2):
        pb = pack_for_logprob(mb, pin=False)
        with torch.no_grad():
            lp, ent = cpu.decoder.logprobs(pb, 1.0)
        off = 0
        for s in mb:
            L = len(s["sample_ids"])
            s["sample_logprobs"] = lp[off:off + L].numpy().copy()
            s["sample_entropies"] = ent[off:off + L].numpy().copy()
            off += L
    for core in (gpu, cpu):
        core.compute_gradients(mb1)
        core.compute_gradients(mb2)
    sg, sc = gpu.apply_gradients(), cpu.apply_gradients()
    assert abs(sg["grad_norm"] - sc["grad_norm"]) < 0.03 * sc["grad_norm"]
    assert abs(sg["loss"] - sc["loss"]) < 5e-3 * max(1.0, abs(sc["loss"]))
    # Adam's first step moves every weight by about lr * sign(g): compare the update direction
    du_g = (gpu.master.cpu() - flat)
    du_c = (cpu.master - flat)
    big = du_c.abs() > 0.5e-3
    agree = (torch.sign(du_g[big]) == torch.sign(du_c[big])).float().mean().item()
    assert agree > 0.97
    assert torch.equal(gpu.params.cpu(), gpu.master.cpu().to(torch.bfloat16))


def test_engine_greedy_tokens_are_oracle_argmax_and_graphs_agree():
    from async_grpo_nccl_b200.engine.engine import RolloutEngine
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.decoder import OracleDecoder
    from async_grpo_nccl_b200.models.layout import ParamLayout

    cfg = PRESETS["tiny128"]
    layout = ParamLayout(cfg)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = (p32 * 3.0).to(torch.bfloat16).to(DEV)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(2, cfg.vocab_size, int(rng.integers(5, 60))).astype(np.int32) for _ in range(6)]
    results = {}
    for graph in (False, True):
        eng = RolloutEngine(cfg, layout, p16, max_seqs=64, max_model_len=512, num_blocks=512, use_cuda_graph=graph)
        for i, pr in enumerate(prompts):
            eng.add_request(i, pr, n=2, max_new_tokens=40, temperature=0.0, seed=i, ignore_eos=True)
        outs = eng.run_until_done()
        eng.check_status()
        assert len(outs) == 12 and eng.sched.num_free_blocks == 512
        results[graph] = {(o.request_id, o.child): o.output_ids for o in outs}
    for k in results[False]:
        assert np.array_equal(results[False][k], results[True][k]), "CUDA-graph replay must reproduce the eager tokens"
    # teacher-forced check: every generated token is the argmax (up to bf16 noise) of (a) the native prefill path,
    # which shares the engine's bf16 numerics but none of its paged-KV / decode kernels, and (b) the fp32 oracle
    from async_grpo_nccl_b200.models.decoder import NativeDecoder
    from async_grpo_nccl_b200.packing import pack_samples

    nat = NativeDecoder(cfg, layout, p16)
    orc = OracleDecoder(cfg, layout, p16.float())
    wl = layout.view(p16.float(), layout.lm_head_name())
    for (rid, child), out_ids in results[False].items():
        if child != 0:
            assert np.array_equal(out_ids, results[False][(rid, 0)])  # greedy children are identical
            continue
        full = np.concatenate([prompts[rid], out_ids])
        pb = pack_samples([{"sample_ids": full, "input_len": len(prompts[rid]), "output_len": len(out_ids)}], pin=False).to_device(DEV)
        with torch.no_grad():
            hn_nat, _, _ = nat.hidden(pb)
            z_nat = hn_nat.float() @ wl.t()
            z_orc = orc.hidden(pb.ids, pb.pos, [0, len(full)]).float() @ wl.t()
        P = len(prompts[rid])
        for j, tok in enumerate(out_ids):
            for z, tol in ((z_nat, 0.03), (z_orc, 0.05)):
                row = z[P - 1 + j]
                top = row.max().item()
                assert row[int(tok)].item() >= top - (tol * abs(top) + 0.05), (rid, j, row[int(tok)].item(), top)


def test_engine_forced_lengths_and_eos():
    from async_grpo_nccl_b200.engine.engine import RolloutEngine
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout

    cfg = PRESETS["tiny128"]
    layout = ParamLayout(cfg)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = (p32 * 3.0).to(torch.bfloat16).to(DEV)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(6, cfg.vocab_size, int(rng.integers(5, 60))).astype(np.int32) for _ in range(6)]
    eng = RolloutEngine(cfg, layout, p16, max_seqs=64, max_model_len=512, num_blocks=512)
    for i, pr in enumerate(prompts):
        eng.add_request(i, pr, n=4, max_new_tokens=100, temperature=1.0, seed=i, forced_new_tokens=[10 + i, 20, 33, 64])
    outs = eng.run_until_done()
    eng.check_status()
    got = {(o.request_id, o.child): o for o in outs}
    for i in range(6):
        for c, want in enumerate([10 + i, 20, 33, 64]):
            o = got[(i, c)]
            assert len(o.output_ids) == want and o.output_ids[-1] == cfg.eos_token_id
    # EOS stopping with one step of read-back lag: sequences end at their first EOS
    eng = RolloutEngine(cfg, layout, p16, max_seqs=64, max_model_len=512, num_blocks=512, eos_token_id=5)
    for i, pr in enumerate(prompts):
        eng.add_request(i, pr, n=8, max_new_tokens=200, temperature=1.0, seed=i)
    outs = eng.run_until_done()
    eng.check_status()
    assert len(outs) == 48
    for o in outs:
        if o.finish_reason == "stop":
            assert o.output_ids[-1] == 5 and (o.output_ids[:-1] != 5).all()
        else:
            # (the 200th token may itself be EOS: the length limit and the stop token then coincide)
            assert len(o.output_ids) == 200 and (o.output_ids[:-1] != 5).all()
    assert eng.sched.num_free_blocks == 512 and eng.sched.num_running == 0


@pytest.mark.parametrize("W,recompute", [(2, False), (4, True)])
def test_fully_sharded_decoder_matches_resident(W, recompute):
    """Sharded weights (gathered per layer, gathers riding on GEMM launches) + scatter sink (weight-gradient GEMMs
    reducing straight into owners' shards) against the resident-parameter path. The W owners are separate buffers of
    this one GPU; every kernel is a single launch, so nothing waits on another launch."""
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.decoder import GradSink, LossConfig, NativeDecoder
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.ops import native
    from async_grpo_nccl_b200.packing import pack_samples
    from async_grpo_nccl_b200.parallel.zero3 import ScatterSink, ShardedWeights

    cfg = PRESETS["tiny128"]
    layout = ParamLayout(cfg, shard_world=W)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = p32.to(torch.bfloat16).to(DEV)
    rng = np.random.default_rng(5)
    pb = pack_samples(_samples(cfg, 12, rng, 100, 300), pin=False).to_device(DEV)  # > 1024 rows: prefetch rides on GEMMs
    assert pb.T >= 1024
    lc = LossConfig(kl_beta=0.0, temperature=1.0)
    ref = NativeDecoder(cfg, layout, p16, recompute=recompute)
    with torch.no_grad():
        lp0, _ = ref.logprobs(pb, 1.0)
    pb.old_logprobs.copy_(lp0 + 0.02 * torch.randn_like(lp0))
    sink_ref = GradSink(layout, DEV)
    stats_ref = ref.forward_backward(pb, lc, 0.5, sink_ref)
    stats_ref = ref.forward_backward(pb, lc, 0.5, sink_ref)  # two microbatches accumulate
    # owners' slices, unit by unit, exactly as a rank of a W-rank job would hold them
    shards16, gshards = [], []
    for r in range(W):
        parts = [p16[gs:gs + ln] for _, gs, ln in layout.local_to_global_ranges(r)]
        shards16.append(torch.cat(parts).contiguous())
        gshards.append(torch.zeros(layout.shard_numel(), dtype=torch.float32, device=DEV))
    C = native()
    weights = ShardedWeights(layout, C, torch.device(DEV), 0, [t.data_ptr() for t in shards16], n_copy=8, chunk_elems=8192)
    weights.invalidate()
    sink = ScatterSink(layout, C, torch.device(DEV), 0, [g.data_ptr() for g in gshards])
    dec = NativeDecoder(cfg, layout, None, recompute=recompute, weights=weights)
    stats = dec.forward_backward(pb, lc, 0.5, sink)
    stats = dec.forward_backward(pb, lc, 0.5, sink)
    torch.cuda.synchronize()
    dec.check_status()
    assert weights.gathers_fused > 0, "no gather rode on a GEMM launch"
    assert torch.allclose(stats, stats_ref, rtol=1e-4, atol=1e-4)
    full = torch.empty_like(p16)
    weights.gather_full(full)
    torch.cuda.synchronize()
    assert torch.equal(full, p16)
    # reassemble the flat gradient from the owners' shards
    got = torch.zeros(layout.total, dtype=torch.float32, device=DEV)
    for r in range(W):
        for lo, gs, ln in layout.local_to_global_ranges(r):
            got[gs:gs + ln] = gshards[r][lo:lo + ln]
    for name in layout.segments:
        a, b = layout.view(got, name), layout.view(sink_ref.flat, name)
        assert (a - b).abs().max().item() <= 5e-3 * b.abs().max().item() + 1e-6, name
    # logprob-only forward through the sharded weights
    lpn, _ = dec.logprobs(pb, 1.0)
    assert (lpn - lp0).abs().max().item() < 1e-5


def test_engine_slot_compaction_does_not_change_tokens(monkeypatch):
    """Sequences finish at different times; moving the survivors into the low slots (so the decode batch shrinks) must
    not change a single sampled token, with EOS stopping and forced lengths alike, eager and with CUDA graphs."""
    from async_grpo_nccl_b200.engine.engine import RolloutEngine
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout

    cfg = PRESETS["tiny128"]
    layout = ParamLayout(cfg)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = (p32 * 3.0).to(torch.bfloat16).to(DEV)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(6, cfg.vocab_size, int(rng.integers(5, 40))).astype(np.int32) for _ in range(12)]
    forced = [[int(x) for x in rng.integers(3, 150, 8)] for _ in range(12)]

    def run(compact, graph, use_forced):
        monkeypatch.setenv("AGRPO_COMPACT_SLOTS", "1" if compact else "0")
        eng = RolloutEngine(cfg, layout, p16, max_seqs=128, max_model_len=512, num_blocks=2048, use_cuda_graph=graph,
                            eos_token_id=5)
        for i, pr in enumerate(prompts):
            # without forced lengths the requests differ in their length limit, so that they end at different times
            eng.add_request(i, pr, n=8, max_new_tokens=120 if use_forced else 10 + 10 * i, temperature=1.0, seed=i,
                            forced_new_tokens=forced[i] if use_forced else None)
        outs = eng.run_until_done()
        eng.check_status()
        assert eng.sched.num_running == 0 and eng.sched.num_free_blocks == 2048
        return {(o.request_id, o.child): (o.output_ids.tolist(), o.finish_reason) for o in outs}, eng.n_compactions

    # Compaction changes the batch size at which a token is computed. Bits are the same across batch sizes within one
    # decode path (the split-K sums have one order whatever the batch), not between the two paths, so each path is
    # pinned in turn: separate kernels only, then the persistent layer kernel for every batch size of this test.
    for mega_rows in ("0", "128"):
        monkeypatch.setenv("AGRPO_MEGA_MAX_ROWS", mega_rows)
        for use_forced in (True, False):
            base, n0 = run(False, False, use_forced)
            assert n0 == 0 and len(base) == 96
            for graph in (False, True):
                got, n = run(True, graph, use_forced)
                assert n > 0, "the workload must trigger at least one compaction"
                assert got == base, f"tokens changed (persistent kernel up to {mega_rows} rows, graph={graph})"


def test_engine_logprobs_agree_with_the_logprob_path():
    """The engine's chosen-token log-probabilities (the probe of vllm_worker.py:286-392) against the values the logprob
    role computes for the same tokens with the training-side kernels: same weights, same temperature."""
    from async_grpo_nccl_b200.engine.engine import RolloutEngine
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.decoder import NativeDecoder
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.packing import pack_for_logprob

    cfg = PRESETS["tiny128"]
    layout = ParamLayout(cfg)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = (p32 * 2.0).to(torch.bfloat16).to(DEV)
    temp = 0.8
    rng = np.random.default_rng(1)
    prompts = [rng.integers(2, cfg.vocab_size, int(rng.integers(5, 40))).astype(np.int32) for _ in range(5)]
    for graph in (False, True):
        eng = RolloutEngine(cfg, layout, p16, max_seqs=64, max_model_len=512, num_blocks=512, use_cuda_graph=graph)
        eng.enable_logprobs()
        for i, pr in enumerate(prompts):
            eng.add_request(i, pr, n=2, max_new_tokens=30, temperature=temp, seed=10 + i, ignore_eos=True)
        outs = eng.run_until_done()
        eng.check_status()
        dec = NativeDecoder(cfg, layout, p16)
        for o in outs:
            assert o.output_logprobs is not None and len(o.output_logprobs) == len(o.output_ids) == 30
            pr = prompts[o.request_id]
            full = np.concatenate([pr, o.output_ids])
            pb = pack_for_logprob([{"sample_ids": full, "input_len": len(pr), "output_len": len(o.output_ids)}], pin=False).to_device(DEV)
            with torch.no_grad():
                logp, _ = dec.logprobs(pb, temp)
            want = logp.float().cpu().numpy()[len(pr) - 1: len(pr) - 1 + len(o.output_ids)]  # position p-1 holds token p
            assert np.all(o.output_logprobs <= 1e-4)
            # A random-init decoder amplifies bf16 differences between the decode kernels (paged cache, split-K order) and
            # the packed prefill kernels from token to token, so single values can be a few tenths apart; the first
            # token comes from the same prefill kernels and must agree closely, the rest must agree as a set.
            diff = np.abs(o.output_logprobs - want)
            assert diff[0] < 2e-2, diff[0]
            assert np.median(diff) < 0.06, np.median(diff)
            assert np.corrcoef(o.output_logprobs, want)[0, 1] > 0.95


def test_engine_batches_above_256_rows_run_in_row_chunks():
    """More than 256 running sequences: the fused decode path processes the rows in chunks of 256 per layer. Every greedy
    token must still be the (bf16-noise tolerant) argmax of the teacher-forced prefill logits."""
    from async_grpo_nccl_b200.engine.engine import RolloutEngine
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.decoder import NativeDecoder
    from async_grpo_nccl_b200.models.layout import ParamLayout
    from async_grpo_nccl_b200.packing import pack_samples

    cfg = PRESETS["tiny128"]
    layout = ParamLayout(cfg)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = (p32 * 3.0).to(torch.bfloat16).to(DEV)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(2, cfg.vocab_size, int(rng.integers(4, 30))).astype(np.int32) for _ in range(150)]
    eng = RolloutEngine(cfg, layout, p16, max_seqs=320, max_model_len=128, num_blocks=2600, use_cuda_graph=True)
    for i, pr in enumerate(prompts):
        eng.add_request(i, pr, n=2, max_new_tokens=10, temperature=0.0, seed=i, ignore_eos=True)
    outs = eng.run_until_done()
    eng.check_status()
    assert len(outs) == 300 and eng.sched.num_free_blocks == 2600
    assert eng.fused_decode and eng.fused_rows == 320 and eng.fused_chunk == 256
    nat = NativeDecoder(cfg, layout, p16)
    wl = layout.view(p16.float(), layout.lm_head_name())
    for o in outs[::7]:
        pr = prompts[o.request_id]
        full = np.concatenate([pr, o.output_ids])
        pb = pack_samples([{"sample_ids": full, "input_len": len(pr), "output_len": len(o.output_ids)}], pin=False).to_device(DEV)
        with torch.no_grad():
            hn, _, _ = nat.hidden(pb)
            z = hn.float() @ wl.t()
        for j, tok in enumerate(o.output_ids):
            row = z[len(pr) - 1 + j]
            top2 = row.topk(2)
            top = top2.values[0].item()
            # the decode path and the teacher-forced pass round differently: a near-tie may go to the runner-up
            assert int(tok) in top2.indices.tolist() or row[int(tok)].item() >= top - (0.03 * abs(top) + 0.05), (o.request_id, j)


def test_engine_prefix_cache_hits_do_not_change_tokens():
    """Prefix caching across requests: prompts that start with an already prefilled chain reuse its KV blocks and only
    compute their remaining tokens. Tokens must equal those of an engine without the cache (greedy and sampled), the
    hit counters must show the reuse, and a weight update must empty the cache."""
    from async_grpo_nccl_b200.engine.engine import RolloutEngine
    from async_grpo_nccl_b200.models.config import PRESETS
    from async_grpo_nccl_b200.models.layout import ParamLayout

    cfg = PRESETS["tiny128"]
    layout = ParamLayout(cfg)
    p32 = torch.empty(layout.total)
    layout.init_random_(p32, 0)
    p16 = (p32 * 3.0).to(torch.bfloat16).to(DEV)
    rng = np.random.default_rng(11)
    prefix = rng.integers(6, cfg.vocab_size, 48).astype(np.int32)
    pa = np.concatenate([prefix, rng.integers(6, cfg.vocab_size, 10).astype(np.int32)])
    pb = np.concatenate([prefix, rng.integers(6, cfg.vocab_size, 23).astype(np.int32)])
    other = rng.integers(6, cfg.vocab_size, 37).astype(np.int32)

    def run(cache):
        eng = RolloutEngine(cfg, layout, p16, max_seqs=32, max_model_len=256, num_blocks=512, use_cuda_graph=False,
                            prefix_caching=cache)
        outs = {}
        eng.add_request("a", pa, n=2, max_new_tokens=8, temperature=0.0, seed=1, ignore_eos=True)
        for o in eng.run_until_done():
            outs[(o.request_id, o.child)] = o.output_ids.tolist()
        first_hits = eng.prefix_hit_tokens
        # the same chain again (whole prompt known: its last block is recomputed), a longer prompt on the same prefix,
        # and an unrelated prompt, prefilled together
        eng.add_request("a2", pa, n=1, max_new_tokens=8, temperature=1.0, seed=2, ignore_eos=True)
        eng.add_request("b", pb, n=2, max_new_tokens=8, temperature=0.0, seed=3, ignore_eos=True)
        eng.add_request("c", other, n=1, max_new_tokens=8, temperature=0.0, seed=4, ignore_eos=True)
        for o in eng.run_until_done():
            outs[(o.request_id, o.child)] = o.output_ids.tolist()
        eng.check_status()
        assert eng.sched.num_running == 0 and eng.sched.num_free_blocks == 512
        return outs, first_hits, eng

    base, h0, _ = run(False)
    got, h1, eng = run(True)
    assert h0 == 0 and h1 == 0
    assert eng.prefix_hit_tokens == 48 + 48, eng.prefix_hit_tokens
    assert got == base
    assert eng.sched.num_cached_blocks > 0
    eng.update_weights_done()
    assert eng.sched.num_cached_blocks == 0
    eng.add_request("a3", pa, n=1, max_new_tokens=4, temperature=0.0, seed=1, ignore_eos=True)
    eng.run_until_done()
    assert eng.prefix_hit_tokens == 96
