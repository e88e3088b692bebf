"""Component benchmarks (device-timed with CUDA events, warm-up first, inputs larger than L2 or L2 flushed between runs).

    python -m async_grpo_nccl_b200.utils.microbench gemm
    python -m async_grpo_nccl_b200.utils.microbench attn
    python -m async_grpo_nccl_b200.utils.microbench lmhead
    python -m async_grpo_nccl_b200.utils.microbench decode --batch 128 --context 1024 --steps 20 [--graph]
    python -m async_grpo_nccl_b200.utils.microbench train --tokens 16384
    python -m async_grpo_nccl_b200.utils.microbench elementwise
    python -m async_grpo_nccl_b200.utils.microbench fused --tokens 16384
    python -m async_grpo_nccl_b200.utils.microbench one --kernel attn_fwd      (small case for an ncu capture)
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29777 \
        -m async_grpo_nccl_b200.utils.microbench sync --trainers 1 --model qwen2.5-1.5b,qwen2.5-7b

Each line of output is a JSON record with the achieved rate and, where a library kernel exists in the image
(cuBLAS through torch.matmul, flash-attn 2), the same measurement for it. Roofline denominators: ``--peak-hbm-gbs`` and
``--peak-bf16-tflops`` (or the environment variables AGRPO_PEAK_HBM_GBS / AGRPO_PEAK_BF16_TFLOPS, or a JSON file with
the keys ``hbm_gbs`` / ``bf16_tflops`` named by AGRPO_PEAKS_FILE); without any of them 6650 GB/s and 1590 TFLOP/s, a
copy / cuBLAS measurement on a B200, marked "fallback" in the records.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import numpy as np
import torch


_PEAK_FLAGS: dict = {}


def _peaks():
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    p = os.environ.get("AGRPO_PEAKS_FILE")
    if p and os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        for k in ("hbm_gbs", "bf16_tflops"):
            if d.get(k):
                out[k], out["source"] = float(d[k]), "measured"
    for k, env in (("hbm_gbs", "AGRPO_PEAK_HBM_GBS"), ("bf16_tflops", "AGRPO_PEAK_BF16_TFLOPS")):
        v = _PEAK_FLAGS.get(k) or os.environ.get(env)
        if v:
            out[k], out["source"] = float(v), "measured"
    return out


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def timeit(fn, iters=10, warmup=3, flush=False):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def out(rec):
    print(json.dumps(rec), flush=True)


def bench_gemm(args):
    from ..ops import native

    C = native()
    pk = _peaks()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    shapes = [(8192, 8192, 8192, False, False), (32768, 2048, 1536, False, False), (32768, 17920, 1536, False, False),
              (32768, 1536, 8960, False, False), (32768, 1536, 8960, False, True), (1536, 8960, 32768, True, True),
              (128, 2048, 1536, False, False), (128, 1536, 1536, False, False), (128, 17920, 1536, False, False),
              (128, 1536, 8960, False, False), (256, 2048, 1536, False, False), (256, 17920, 1536, False, False),
              (256, 1536, 8960, False, False)]
    for M, N, K, am, bm in shapes:
        a = torch.randn((K, M) if am else (M, K), device="cuda", dtype=torch.bfloat16)
        b = torch.randn((K, N) if bm else (N, K), device="cuda", dtype=torch.bfloat16)
        d = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        A, B = (a.t() if am else a), (b.t() if bm else b)
        small = M <= 512
        t = timeit(lambda: C.gemm_bf16(a, b, d, am, bm, None, 1.0, False, st, None), flush=small)
        t2 = timeit(lambda: torch.matmul(A, B.t(), out=d), flush=small)
        fl = 2.0 * M * N * K
        rec = {"bench": "gemm", "M": M, "N": N, "K": K, "a_mn": am, "b_mn": bm, "ms": t, "tflops": fl / t / 1e9,
               "cublas_ms": t2, "cublas_tflops": fl / t2 / 1e9, "frac_of_peak": fl / t / 1e9 / pk["bf16_tflops"], "peak": pk["source"]}
        if small:
            rec["weight_gbs"] = N * K * 2 / t / 1e6
            rec["frac_of_hbm"] = rec["weight_gbs"] / pk["hbm_gbs"]
        out(rec)
    assert int(st.item()) == 0


def bench_fused(args):
    """Fused compute + collective kernels on ONE GPU, the owners being separate local buffers: measures what the copier
    CTAs and the reduce-scatter epilogue cost next to the plain kernels. With --world > 1 under torchrun the same
    kernels run over real peer memory (symmetric allocations)."""
    from ..ops import native

    C = native()
    pk = _peaks()
    W = 4
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    T, H, F = args.tokens, 1536, 8960
    unit_n = (46_800_000 // (128 * W)) * 128 * W        # one Qwen2.5-1.5B block
    n_per = unit_n // W
    shards = [torch.randn(n_per, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    staging = torch.empty(unit_n, device="cuda", dtype=torch.bfloat16)
    chunk = 1 << 18
    flags = torch.zeros((unit_n + chunk - 1) // chunk, dtype=torch.int64, device="cuda")
    ptrs = [s_.data_ptr() for s_ in shards]
    a = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(2 * F, H, device="cuda", dtype=torch.bfloat16)
    d = torch.empty(T, 2 * F, device="cuda", dtype=torch.bfloat16)
    ep = [0]

    def fused(n_copy):
        ep[0] += 1
        C.ag_gemm(a, b, d, False, False, None, False, st, None, src_ptrs=ptrs, my_rank=0, staging=staging, n_per_owner=n_per,
                  flags=flags, epoch=ep[0], chunk_elems=chunk, n_copy=n_copy)

    def serial():
        ep[0] += 1
        C.unit_gather(ptrs, 0, staging, n_per, flags, ep[0], chunk, 64)
        C.gemm_bf16(a, b, d, False, False, None, 1.0, False, st, None)

    def gather_only():
        ep[0] += 1
        C.unit_gather(ptrs, 0, staging, n_per, flags, ep[0], chunk, 64)

    t_plain = timeit(lambda: C.gemm_bf16(a, b, d, False, False, None, 1.0, False, st, None))
    t_gather = timeit(gather_only)
    t_serial = timeit(serial)
    fl = 2.0 * T * 2 * F * H
    for n_copy in (2, 4, 8, 16):
        t = timeit(lambda: fused(n_copy))
        out({"bench": "ag_gemm_prefetch", "M": T, "N": 2 * F, "K": H, "unit_mb": unit_n * 2 / 1e6, "n_copy": n_copy, "ms": t,
             "gemm_alone_ms": t_plain, "gather_alone_ms": t_gather, "serial_ms": t_serial, "hidden_frac": (t_serial - t) / t_gather,
             "tflops": fl / t / 1e9, "gather_gbs": unit_n * 2 / t_gather / 1e6})
    # the GEMM consumes the unit being gathered (tile-by-tile waits)
    rel = 4096
    bview = staging[rel: rel + 2 * F * H].view(2 * F, H)

    def fused_self():
        ep[0] += 1
        C.ag_gemm(a, bview, d, False, False, None, False, st, None, src_ptrs=ptrs, my_rank=0, staging=staging, n_per_owner=n_per,
                  flags=flags, epoch=ep[0], chunk_elems=chunk, n_copy=16)

    t = timeit(fused_self)
    out({"bench": "ag_gemm_consume", "M": T, "N": 2 * F, "K": H, "ms": t, "gemm_alone_ms": t_plain, "gather_alone_ms": t_gather,
         "serial_ms": t_serial})
    # weight gradient: local fp32 accumulate vs reduce-scatter epilogue
    dy = torch.randn(T, 2 * F, device="cuda", dtype=torch.bfloat16)
    acc = torch.zeros(2 * F, H, device="cuda", dtype=torch.float32)
    gsh = [torch.zeros(n_per, device="cuda", dtype=torch.float32) for _ in range(W)]
    gp = [g.data_ptr() for g in gsh]
    t_acc = timeit(lambda: C.gemm_bf16(dy, a, acc, True, True, None, 1.0, True, st, None))
    t_rs = timeit(lambda: C.gemm_rs(dy, a, True, True, 1.0, gp, n_per, rel, H, st))
    out({"bench": "gemm_rs", "M": 2 * F, "N": H, "K": T, "ms": t_rs, "local_accumulate_ms": t_acc, "tflops": fl / t_rs / 1e9,
         "local_tflops": fl / t_acc / 1e9, "frac_of_peak": fl / t_rs / 1e9 / pk["bf16_tflops"], "peak": pk["source"]})
    torch.cuda.synchronize()
    assert int(st.item()) == 0


def bench_sync(args):
    """Trainer -> inference weight sync (run under torchrun, one rank per GPU). For every (t, r) of ``--pairs`` the first t
    ranks hold the FSDP shards and the next r ranks receive; the remaining ranks only take part in the barriers. Per model
    it times, on the device and as the max over ranks:
      * the peer-memory push with plain peer stores and, when the allocation has a multicast address, with ``multimem.st``;
      * an NCCL broadcast per shard range;
      * the reference's pattern (gpu_process_worker.py:1609-1637): per parameter tensor an all-gather inside the trainer
        group (``full_tensor()``), a copy into a fresh tensor on trainer rank 0 and one broadcast over every GPU worker.
    """
    import math

    import torch.distributed as dist

    from ..models.config import PRESETS
    from ..models.layout import ParamLayout
    from ..ops import native
    from ..parallel import symm

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl")
    C = native()
    if args.pairs:
        pairs = [tuple(int(x) for x in p.split(",")) for p in args.pairs.split(";")]
    else:
        t0 = max(1, min(args.trainers, world - 1))
        pairs = [(t0, world - t0)]
    pairs = [(t, r) for t, r in pairs if t + r <= world]
    lcm = 1
    for t, _ in pairs:
        lcm = lcm * t // math.gcd(lcm, t)

    def timed(fn, iters=3):
        best = []
        for i in range(iters + 1):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 1:
                best.append(e0.elapsed_time(e1))
        ms = torch.tensor([sorted(best)[len(best) // 2]], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for model in args.model.split(","):
        cfg = PRESETS[model]
        layout = ParamLayout(cfg, shard_world=lcm)  # every unit divides evenly by each t of the sweep
        flags = symm.alloc_symmetric(128, torch.int64, dev, dist.group.WORLD)
        dst = symm.alloc_symmetric(layout.total, torch.bfloat16, dev, dist.group.WORLD)
        src_full = torch.empty(layout.total, device=dev, dtype=torch.bfloat16)
        torch.manual_seed(1234)  # the same values on every rank: a receiver can check what it got bit for bit
        src_full.normal_(0, 0.02)
        gb = layout.total * 2 / 1e9
        for t, r in pairs:
            trainers, infer = list(range(t)), list(range(t, t + r))
            members = trainers + infer
            tg = dist.new_group(trainers)
            sg = dist.new_group(members)

            class _Plane:  # the two buffers a weight sync needs
                pass

            pl = _Plane()
            pl.layout, pl.C, pl.trainer_ranks, pl.infer_ranks, pl.my_rank, pl.device = layout, C, trainers, infer, rank, dev
            pl.flags, pl.infer_params = flags, dst
            ti = trainers.index(rank) if rank in trainers else None
            src = src_full if rank in trainers else None
            res = {"bench": "weight_sync", "model": model, "trainers": t, "receivers": r, "param_gb": gb}
            for mode in ("plain", "multicast"):
                os.environ["AGRPO_MULTICAST"] = "1" if mode == "multicast" else "0"
                torch.cuda.synchronize()
                dist.barrier()
                flags.local.zero_()  # a new sync object counts its barrier epochs from zero again
                dst.local.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                ws = symm.WeightSync(pl)
                if mode == "multicast" and not ws.dst_mc:
                    res["peer_push_multicast_ms"] = None
                    continue
                ms = timed(lambda: ws.push(src, ti))
                ws.pg.check()
                res[f"peer_push_{mode}_ms"] = ms
                if rank in infer:  # bit-exact: the receivers hold exactly the source's bf16 values
                    assert torch.equal(dst.local, src_full), f"weight push ({mode}) did not deliver the source bit for bit"
            os.environ["AGRPO_MULTICAST"] = "1"
            if rank in members:
                def shard_ranges():
                    symm.broadcast_weights(src if src is not None else dst.local, layout, sg, trainers, ti,
                                           dst.local if rank in infer else None)
            else:
                def shard_ranges():
                    return None
            res["nccl_broadcast_per_shard_range_ms"] = timed(shard_ranges)

            def reference_pattern():
                if rank not in members:
                    return
                for seg in layout.segments.values():
                    m = seg.numel
                    if rank in trainers:
                        mt = (m + t - 1) // t
                        if t > 1:
                            full = torch.empty(mt * t, dtype=torch.bfloat16, device=dev)
                            lo = min(seg.offset + ti * mt, layout.total - mt)
                            dist.all_gather_into_tensor(full, src_full[lo:lo + mt], group=tg)
                        else:
                            full = src_full[seg.offset:seg.offset + m]
                    tensor = torch.empty(m, dtype=torch.bfloat16, device=dev)
                    if rank == 0:
                        tensor.copy_(full[:m])
                    dist.broadcast(tensor, src=0, group=sg)

            res["reference_pattern_ms"] = timed(reference_pattern, iters=2)
            res["tensors"] = len(layout.segments)
            if rank == 0:
                push = min(x for x in (res.get("peer_push_plain_ms"), res.get("peer_push_multicast_ms")) if x)
                res.update({"best_push_gbs_into_each_receiver": gb / push * 1e3, "receiver_ingress_bound_ms_at_770": gb / 770.0 * 1e3,
                            "source_egress_bound_ms_plain_at_770": gb * r / t / 770.0 * 1e3,
                            "speedup_vs_reference_pattern": res["reference_pattern_ms"] / push})
                out(res)
            dist.destroy_process_group(tg)
            dist.destroy_process_group(sg)
        del dst, src_full, flags
        torch.cuda.empty_cache()
    dist.destroy_process_group()


def bench_one(args):
    """One kernel, three launches, a small case (operands of a few hundred MB at most): the program to put under
    `ncu --set full -k regex:<kernel> -c 2`. Prints the device time of the third launch."""
    from ..ops import native

    C = native()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    dev, bf = "cuda", torch.bfloat16
    k = args.kernel
    if k == "gemm":
        a = torch.randn(8192, 8192, device=dev, dtype=bf)
        b = torch.randn(8192, 8192, device=dev, dtype=bf)
        d = torch.empty(8192, 8192, device=dev, dtype=bf)
        fn = lambda: C.gemm_bf16(a, b, d, False, False, None, 1.0, False, st, None)
    elif k in ("attn_fwd", "attn_bwd"):
        Hq, Hkv, D, lens = 12, 2, 128, [8192, 8192]
        T, Cc = sum(lens), (Hq + 2 * Hkv) * D
        qkv = torch.randn(T, Cc, device=dev).to(bf)
        o = torch.zeros(T, Hq * D, device=dev, dtype=bf)
        lse = torch.zeros(Hq, T, device=dev)
        tiles = _tiles(lens)
        sc = 1 / math.sqrt(D)
        C.attn_varlen_fwd(qkv, o, lse, tiles, Hq, Hkv, D, sc, st)
        if k == "attn_fwd":
            fn = lambda: C.attn_varlen_fwd(qkv, o, lse, tiles, Hq, Hkv, D, sc, st)
        else:
            dout = torch.randn(T, Hq * D, device=dev).to(bf)
            delta, dq_acc = torch.empty(Hq, T, device=dev), torch.empty(T, Hq * D, device=dev)
            dqkv = torch.zeros(T, Cc, device=dev, dtype=bf)
            fn = lambda: C.attn_varlen_bwd(qkv, o, dout, lse, delta, dq_acc, dqkv, tiles, Hq, Hkv, D, sc, st)
    elif k in ("lmhead_fwd", "lmhead_bwd"):
        T, H, V = 8192, 1536, 151936
        h = torch.randn(T, H, device=dev).to(bf)
        W = (torch.randn(V, H, device=dev) * 0.02).to(bf)
        labels = torch.randint(0, V, (T,), device=dev, dtype=torch.int32)
        groups = C.lmhead_num_groups(V, T)
        partials, ll = torch.empty(3 * groups * T, device=dev), torch.zeros(T, device=dev)
        logp, ent, lse = (torch.empty(T, device=dev) for _ in range(3))
        C.lmhead_logprob(h, W, labels, 1.0, partials, ll, logp, ent, lse, st)
        if k == "lmhead_fwd":
            fn = lambda: C.lmhead_logprob(h, W, labels, 1.0, partials, ll, logp, ent, lse, st)
        else:
            dlogp = torch.randn(T, device=dev) / T
            dz = torch.empty(T, 4096, device=dev, dtype=bf)
            dh, dW = torch.empty(T, H, device=dev), torch.zeros(V, H, device=dev)
            fn = lambda: C.lmhead_backward(h, W, labels, lse, dlogp, 1.0, dz, dh, dW, st)
    elif k in ("splitk", "swiglu"):
        M, H, F = 128, 1536, 8960
        x = torch.randn(M, F if k == "splitk" else H, device=dev, dtype=bf)
        ss = torch.full((M,), int(H) << 30, device=dev, dtype=torch.int64)
        if k == "splitk":
            w, d = torch.randn(H, F, device=dev, dtype=bf), torch.empty(M, H, device=dev, dtype=bf)
            res = torch.randn(M, H, device=dev, dtype=bf)
            sso = torch.zeros(M, device=dev, dtype=torch.int64)
            fn = lambda: C.gemm_decode(x, w, d, None, res, None, sso, 1e-6, st)
        else:
            w, d = torch.randn(2 * F, H, device=dev, dtype=bf), torch.empty(M, F, device=dev, dtype=bf)
            fn = lambda: C.gemm_swiglu(x, w, d, ss, 1e-6, st)
    elif k == "gemm_rs":
        T, No, Ki, W = 16384, 17920, 1536, 4
        n_per = (No * Ki + 4096 + 128 * W - 1) // (128 * W) * 128
        dy, x = torch.randn(T, No, device=dev, dtype=bf), torch.randn(T, Ki, device=dev, dtype=bf)
        sh = [torch.zeros(n_per, device=dev) for _ in range(W)]
        ptrs = [t.data_ptr() for t in sh]
        fn = lambda: C.gemm_rs(dy, x, True, True, 1.0, ptrs, n_per, 4096, Ki, st)
    else:
        raise SystemExit(f"unknown kernel {k}")
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    out({"bench": "one", "kernel": k, "ms": e0.elapsed_time(e1)})


def _tiles(lens):
    tiles, start = [], 0
    for L in lens:
        for q0 in range(0, L, 128):
            tiles.append((start, L, q0, 0))
        start += L
    tiles.sort(key=lambda t: -t[2])
    return torch.tensor(tiles, dtype=torch.int32, device="cuda")


def bench_attn(args):
    from ..ops import native

    C = native()
    pk = _peaks()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    Hq, Hkv, D = 12, 2, 128
    for lens in ([4096] * 8, [16384] * 2, [512] * 64, [2048] * 16):
        T, Cc = sum(lens), (Hq + 2 * Hkv) * D
        qkv = torch.randn(T, Cc, device="cuda").to(torch.bfloat16)
        dout = torch.randn(T, Hq * D, device="cuda").to(torch.bfloat16)
        o = torch.zeros(T, Hq * D, device="cuda", dtype=torch.bfloat16)
        lse = torch.zeros(Hq, T, device="cuda")
        tiles = _tiles(lens)
        sc = 1 / math.sqrt(D)
        tf = timeit(lambda: C.attn_varlen_fwd(qkv, o, lse, tiles, Hq, Hkv, D, sc, st))
        delta, dq_acc = torch.empty(Hq, T, device="cuda"), torch.empty(T, Hq * D, device="cuda")
        dqkv = torch.zeros(T, Cc, device="cuda", dtype=torch.bfloat16)
        tb = timeit(lambda: C.attn_varlen_bwd(qkv, o, dout, lse, delta, dq_acc, dqkv, tiles, Hq, Hkv, D, sc, st))
        flf = sum(4.0 * L * L / 2 * Hq * D for L in lens)
        rec = {"bench": "attn_varlen", "lens": f"{lens[0]}x{len(lens)}", "Hq": Hq, "Hkv": Hkv, "D": D, "fwd_ms": tf,
               "fwd_tflops": flf / tf / 1e9, "bwd_ms": tb, "bwd_tflops": 2.5 * flf / tb / 1e9,
               "fwd_frac_of_peak": flf / tf / 1e9 / pk["bf16_tflops"], "peak": pk["source"]}
        try:
            from flash_attn import flash_attn_varlen_func

            q = qkv[:, :Hq * D].reshape(T, Hq, D).clone().requires_grad_(True)
            k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D).clone().requires_grad_(True)
            v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D).clone().requires_grad_(True)
            cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device="cuda")
            t2 = timeit(lambda: flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True))
            oo = flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True)
            do = dout.view(T, Hq, D)
            t3 = timeit(lambda: torch.autograd.grad(oo, (q, k, v), do, retain_graph=True))
            rec.update(fa2_fwd_ms=t2, fa2_fwd_tflops=flf / t2 / 1e9, fa2_bwd_ms=t3, fa2_bwd_tflops=2.5 * flf / t3 / 1e9)
        except Exception as e:  # flash-attn not importable
            rec["fa2"] = repr(e)
        out(rec)
    assert int(st.item()) == 0


def bench_lmhead(args):
    from ..ops import native

    C = native()
    pk = _peaks()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    H, V = 1536, 151936
    for T in (4096, 16384):
        h = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        W = (torch.randn(V, H, device="cuda") * 0.02).to(torch.bfloat16)
        labels = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
        groups = C.lmhead_num_groups(V, T)
        partials, ll = torch.empty(3 * groups * T, device="cuda"), torch.zeros(T, device="cuda")
        logp, ent, lse = (torch.empty(T, device="cuda") for _ in range(3))
        dlogp = torch.randn(T, device="cuda") / T
        dz = torch.empty(T, 4096, device="cuda", dtype=torch.bfloat16)
        dh, dW = torch.empty(T, H, device="cuda"), torch.zeros(V, H, device="cuda")
        tf = timeit(lambda: C.lmhead_logprob(h, W, labels, 1.0, partials, ll, logp, ent, lse, st), iters=5)
        tb = timeit(lambda: C.lmhead_backward(h, W, labels, lse, dlogp, 1.0, dz, dh, dW, st), iters=5)

        def torch_fwd():
            for s in range(0, T, 2048):
                z = (h[s:s + 2048] @ W.t()).float()
                torch.logsumexp(z, -1)
                z.gather(1, labels[s:s + 2048].long()[:, None])

        tt = timeit(torch_fwd, iters=3)
        fl = 2.0 * T * H * V
        out({"bench": "lmhead_loss", "T": T, "H": H, "V": V, "fwd_ms": tf, "fwd_tflops": fl / tf / 1e9, "bwd_ms": tb,
             "bwd_tflops": 3 * fl / tb / 1e9, "torch_chunked_fwd_ms": tt, "fwd_frac_of_peak": fl / tf / 1e9 / pk["bf16_tflops"],
             "peak": pk["source"]})
    assert int(st.item()) == 0


def bench_elementwise(args):
    from ..ops import native

    C = native()
    pk = _peaks()
    T, H, F = 32768, 1536, 8960
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    y, rstd = torch.empty_like(x), torch.empty(T, device="cuda")
    t = timeit(lambda: C.rmsnorm_fwd(x, w, y, rstd, 1e-6))
    out({"bench": "rmsnorm_fwd", "T": T, "H": H, "ms": t, "gbs": 2 * T * H * 2 / t / 1e6, "frac_of_hbm": 2 * T * H * 2 / t / 1e6 / pk["hbm_gbs"]})
    gu = torch.randn(T, 2 * F, device="cuda").to(torch.bfloat16)
    act = torch.empty(T, F, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: C.swiglu_fwd(gu, act))
    out({"bench": "swiglu_fwd", "T": T, "F": F, "ms": t, "gbs": 3 * T * F * 2 / t / 1e6, "frac_of_hbm": 3 * T * F * 2 / t / 1e6 / pk["hbm_gbs"]})
    n = 1_543_000_000 // 4
    p, m, v, g = (torch.zeros(n, device="cuda") for _ in range(4))
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ns = torch.ones(1, device="cuda")
    t = timeit(lambda: C.adamw_step(p, m, v, g, p16, 1e-6, 0.9, 0.999, 1e-8, 0.0, 1, 1.0, ns, 1.0, True), iters=5)
    by = n * (4 * 4 + 4 * 4 + 2)
    out({"bench": "adamw", "n": n, "ms": t, "gbs": by / t / 1e6, "frac_of_hbm": by / t / 1e6 / pk["hbm_gbs"]})


def _engine(args, graph):
    from ..engine.engine import RolloutEngine
    from ..models.config import PRESETS
    from ..models.layout import ParamLayout

    cfg = PRESETS[args.model]
    layout = ParamLayout(cfg)
    tp = None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # launched with torch.distributed.run: the ranks form ONE tensor-parallel engine replica
        import torch.distributed as dist

        from ..ops import native
        from ..parallel import symm

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        if not dist.is_initialized():
            dist.init_process_group("nccl")
        tp = symm.TensorParallelComm(list(range(world)), dist.get_rank(), min(256, max(64, args.batch)), cfg.hidden_size,
                                     torch.device("cuda", torch.cuda.current_device()), native())
    params = torch.empty(layout.total, dtype=torch.bfloat16, device="cuda")
    layout.init_random_device_(params, 0)  # same seed on every rank: identical parameters
    eng = RolloutEngine(cfg, layout, params, max_seqs=max(64, args.batch), max_model_len=args.context + args.steps + 64,
                        num_blocks=(args.batch * (args.context + args.steps + 64)) // 16 + 1024, use_cuda_graph=graph, tp=tp)
    return cfg, eng


def bench_decode(args):
    pk = _peaks()
    cfg, eng = _engine(args, args.graph)
    rng = np.random.default_rng(0)
    n = 8
    for i in range(args.batch // n):
        eng.add_request(i, rng.integers(0, cfg.vocab_size, args.context).astype(np.int32), n=n, max_new_tokens=args.steps + 8,
                        temperature=1.0, seed=i, forced_new_tokens=[args.steps + 8] * n)
    while eng.sched.num_waiting > 0 or eng.pending:
        eng.step()  # prefill
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        eng.step()
    e1.record()
    torch.cuda.synchronize()
    eng.check_status()
    ms = e0.elapsed_time(e1) / args.steps
    tp_size = eng.tp_size
    if tp_size > 1:
        import torch.distributed as dist

        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # device time, max over the replica's ranks
        ms = float(t.item())
        if dist.get_rank() != 0:
            dist.barrier()
            dist.destroy_process_group()
            return
    # bytes one rank streams per step: its share of the layer matrices and of the KV cache, plus the replicated lm_head
    head = cfg.vocab_size * cfg.hidden_size * 2
    layout_bytes = (eng.layout.total * 2 - head * (1 if cfg.tie_word_embeddings else 2)) // tp_size + head
    kv_bytes = (args.batch * (args.context + args.steps // 2) * cfg.num_hidden_layers * 2 * cfg.num_key_value_heads * cfg.head_dim * 2
                // tp_size)
    out({"bench": "decode_step", "model": args.model, "batch": args.batch, "context": args.context, "graph": bool(args.graph),
         "tensor_parallel": tp_size,
         "ms_per_step": ms, "tokens_per_s": args.batch / ms * 1e3, "weight_bytes": layout_bytes, "kv_bytes": kv_bytes,
         "ideal_ms": (layout_bytes + kv_bytes) / pk["hbm_gbs"] / 1e6, "frac_of_hbm": (layout_bytes + kv_bytes) / ms / 1e6 / pk["hbm_gbs"],
         "peak": pk["source"]})
    if tp_size > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if getattr(args, "trace", False) and getattr(eng, "mega_rows", 0):
        # clock64 stamps of CTA 0 in one middle layer, microseconds from the layer's start (1965 MHz assumed)
        eng.use_cuda_graph = False
        eng.mega_trace = torch.zeros(32 + 4 * 160, dtype=torch.int64, device="cuda")
        eng.mega_trace_layer = cfg.num_hidden_layers // 2
        eng.step()
        torch.cuda.synchronize()
        t = eng.mega_trace.cpu().numpy().astype(np.float64)
        names = ["mma_first_operands", "mma_committed", "acc_ready", "partial_stored", "splits_arrived", "share_done"]
        rel = lambda i: round((t[i] - t[26]) / 1965.0, 2) if t[i] > 0 else None
        rec = {"bench": "decode_layers_trace", "layer": eng.mega_trace_layer, "unit": "us since the layer's start on CTA 0"}
        for ph, pn in enumerate(["qkv", "o", "gate_up", "down"]):
            rec[pn] = {n: rel(ph * 6 + i) for i, n in enumerate(names)}
        rec["attention"] = {"inputs_ready": rel(24), "end": rel(25)}
        per = t[32:].reshape(-1, 4)
        per = per[per[:, 0] > 0]
        if len(per):
            t0 = per[:, 3][per[:, 3] > 0].min() if (per[:, 3] > 0).any() else per[:, 0].min()
            us = lambda col: [round(float(x), 2) for x in ((np.percentile(col[col > 0], [0, 50, 100]) - t0) / 1e3)]
            rec["all_ctas_us_min_med_max"] = {"qkv_first_mma": us(per[:, 3]), "attention_inputs_ready": us(per[:, 0]),
                                              "attention_end": us(per[:, 1]), "o_first_mma": us(per[:, 2])}
        out(rec)


def bench_train(args):
    from ..config import make_config
    from ..models.config import PRESETS
    from ..roles.trainer import TrainerCore

    pk = _peaks()
    mcfg = PRESETS[args.model]
    cfg = make_config({"model_name_or_path": args.model, "train_minibatch_sample_size": 8, "global_num_verifiers": 0,
                       "activation_recompute": "full" if args.recompute else "none"})
    from ..launch import initial_weights
    from ..models.layout import ParamLayout

    flat = initial_weights(cfg, mcfg, ParamLayout(mcfg), "cuda")
    core = TrainerCore(cfg, mcfg, torch.device("cuda"), init_flat_fp32=flat)
    del flat
    rng = np.random.default_rng(0)
    n = 8
    per = args.tokens // n
    samples = []
    for _ in range(n):
        li = 256
        L = per
        samples.append({"sample_ids": rng.integers(0, mcfg.vocab_size, L).astype(np.int32), "input_len": li, "output_len": L - li,
                        "advantage": float(rng.normal()), "sample_logprobs": np.full(L, -11.9, np.float32),
                        "sample_entropies": np.zeros(L, np.float32), "reward": 1.0})

    def step():
        core.compute_gradients(samples)
        core.apply_gradients()

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.iters
    T = per * n
    nparam = mcfg.num_parameters() - (0 if mcfg.tie_word_embeddings else 0)
    fl = 6.0 * T * (nparam - mcfg.vocab_size * mcfg.hidden_size * (0 if mcfg.tie_word_embeddings else 1))
    fl += 3 * sum(4.0 * per * per / 2 * mcfg.num_attention_heads * mcfg.head_dim for _ in range(n)) * mcfg.num_hidden_layers
    if args.recompute:
        fl *= 4.0 / 3.0
    out({"bench": "train_step", "model": args.model, "tokens": T, "recompute": bool(args.recompute), "ms": ms,
         "tokens_per_s": T / ms * 1e3, "model_tflops": fl / ms / 1e9, "frac_of_peak": fl / ms / 1e9 / pk["bf16_tflops"],
         "peak": pk["source"], "max_mem_gb": torch.cuda.max_memory_allocated() / 1e9})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn", "lmhead", "elementwise", "decode", "train", "fused", "one", "sync"])
    ap.add_argument("--kernel", default="gemm", help="for 'one': gemm | attn_fwd | attn_bwd | lmhead_fwd | lmhead_bwd | splitk | "
                    "swiglu | gemm_rs")
    ap.add_argument("--trainers", type=int, default=1, help="for 'sync': ranks that hold shards (the rest receive)")
    ap.add_argument("--pairs", default=None, help="for 'sync': (trainers, receivers) pairs to sweep, e.g. '1,1;2,2;4,4;4,3;7,1'")
    ap.add_argument("--model", default="qwen2.5-1.5b")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--trace", action="store_true", help="decode: print the phase stamps of the persistent layer kernel (one eager step)")
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--peak-hbm-gbs", type=float, default=None, help="roofline denominator: measured copy bandwidth, GB/s")
    ap.add_argument("--peak-bf16-tflops", type=float, default=None, help="roofline denominator: measured cuBLAS bf16 TFLOP/s")
    args = ap.parse_args()
    _PEAK_FLAGS.update({"hbm_gbs": args.peak_hbm_gbs, "bf16_tflops": args.peak_bf16_tflops})
    {"gemm": bench_gemm, "attn": bench_attn, "lmhead": bench_lmhead, "elementwise": bench_elementwise, "decode": bench_decode,
     "train": bench_train, "fused": bench_fused, "one": bench_one, "sync": bench_sync}[args.what](args)


if __name__ == "__main__":
    main()
