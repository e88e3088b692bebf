"""C++ continuous-batching scheduler (csrc/host/kv_allocator.cpp) driven from Python, no GPU: admission, block growth,
finish, and slot compaction (running sequences are kept in a dense prefix of the slot range)."""
import numpy as np
import pytest


def _sched(**kw):
    from async_grpo_nccl_b200.ops import have_native, native

    if not have_native():
        pytest.skip("extension not built")
    C = native()  # host-side classes of the extension work without a GPU
    args = dict(num_blocks=256, block_size=16, max_seqs=16, max_blocks_per_seq=32, max_prefill_tokens=4096)
    args.update(kw)
    return C.Scheduler(**args)


def test_admission_decode_growth_and_finish():
    s = _sched()
    s.add_group(0, 20, 4, 40, [])
    s.add_group(1, 5, 2, 40, [])
    plan = s.plan_prefill()
    assert sorted(plan["group_ids"]) == [0, 1] and len(plan["seq_slots"]) == 6
    assert s.num_running == 6 and s.num_free_slots == 10
    free0 = s.num_free_blocks
    d = s.plan_decode()
    assert d["num_active"] == 6 and isinstance(d["active_slots"], np.ndarray) and d["active_slots"].dtype == np.int32
    assert d["batch_rows"] == int(d["active_slots"].max()) + 1
    for _ in range(20):  # cross block boundaries: every sequence gets new blocks through table updates
        d = s.plan_decode()
    assert s.num_free_blocks < free0
    for sid in plan["seq_ids"]:
        s.finish(sid)
    assert s.num_running == 0 and s.num_free_slots == 16 and s.num_free_blocks == 256


def test_compaction_moves_high_slots_into_low_holes():
    s = _sched()
    s.add_group(0, 8, 8, 100, [])
    s.add_group(1, 8, 4, 100, [])
    plan = s.plan_prefill()
    slots = dict(zip(plan["seq_ids"], plan["seq_slots"]))
    assert sorted(slots.values()) == list(range(12))
    # finish the sequences sitting in slots 0, 1, 2 and 5: the survivors in the highest slots move down
    by_slot = {v: k for k, v in slots.items()}
    for sl in (0, 1, 2, 5):
        s.finish(by_slot[sl])
    assert s.highest_slot == 11 and s.num_running == 8
    blocks_before = {sid: s.seq_info(sid)["blocks"] for sid in slots if s.seq_info(sid) is not None}
    moves = s.compact_slots()
    assert sorted(m[0] for m in moves) == [8, 9, 10, 11] and sorted(m[1] for m in moves) == [0, 1, 2, 5]
    assert s.highest_slot == 7
    for frm, to in moves:
        assert s.seq_info(by_slot[frm])["slot"] == to
    # blocks stay with their sequences, and a second compaction has nothing to do
    assert {sid: s.seq_info(sid)["blocks"] for sid in blocks_before} == blocks_before
    assert s.compact_slots() == []
    d = s.plan_decode()
    assert d["batch_rows"] == 8 and sorted(d["active_slots"].tolist()) == list(range(8))
    # the next admission takes the lowest free slots
    s.add_group(2, 8, 2, 10, [])
    p2 = s.plan_prefill()
    assert sorted(p2["seq_slots"]) == [8, 9]


def test_block_pool_exhaustion_preempts_the_youngest_sequence():
    # 6 blocks of 16 tokens: two sequences of 30 prompt tokens take 2 blocks each; both grow until the pool runs dry
    s = _sched(num_blocks=6, max_seqs=4, max_blocks_per_seq=16)
    s.add_group(0, 30, 1, 200, [])
    s.add_group(1, 30, 1, 200, [])
    plan = s.plan_prefill()
    ids = list(plan["seq_ids"])
    assert len(ids) == 2 and s.num_free_blocks == 2
    preempted, steps = [], 0
    while not preempted and steps < 100:
        d = s.plan_decode()
        preempted = list(d["preempted"])
        steps += 1
    assert preempted == [max(ids)], "the youngest running sequence is the victim"
    # the victim's slot and blocks are free again; the survivor keeps generating alone
    assert s.num_running == 1 and d["num_active"] == 1
    assert all(s.seq_info(i) is None or s.seq_info(i)["slot"] >= 0 for i in ids if i != max(ids))
    survivor_slot = s.seq_info(min(ids))["slot"]
    assert d["active_slots"].tolist() == [survivor_slot]
    assert all(int(u) == survivor_slot for u in d["upd_slot"]), "table updates of the evicted sequence are dropped"
    d2 = s.plan_decode()
    assert d2["num_active"] == 1 and list(d2["preempted"]) == []


def test_prefix_cache_reuses_blocks_across_requests_and_evicts_oldest_first():
    """Prefix caching in the scheduler: a prompt whose leading full blocks carry known hashes takes those blocks instead
    of new ones (only after the prefill that fills them has been planned in an EARLIER call), at least one token is
    always left to compute, unused cached blocks count as free and are evicted oldest first, and a cleared cache
    forgets everything."""
    from async_grpo_nccl_b200.ops import native

    C = native()
    bs = 4
    s = C.Scheduler(num_blocks=24, block_size=bs, max_seqs=8, max_blocks_per_seq=16, max_prefill_tokens=1024)
    # request 0: 10 prompt tokens = 2 full blocks (hashes 11, 12) + a tail
    s.add_group(0, 10, 1, 4, [], [11, 12])
    p0 = s.plan_prefill()
    assert p0["cached_lens"] == [0] and len(p0["slot_mapping"]) == 10 and p0["prefix_slots"] == []
    blocks0 = s.seq_info(p0["seq_ids"][0])["blocks"]
    # request 1, planned in the SAME call as request 2 below, shares the chain; request 0's blocks are registered when the
    # next planning call starts
    s.add_group(1, 9, 2, 4, [], [11, 12])
    s.add_group(2, 8, 1, 4, [], [11, 12])   # exactly 2 full blocks: the last one is recomputed (one token at least)
    p1 = s.plan_prefill()
    assert p1["cached_lens"] == [8, 4]
    assert len(p1["slot_mapping"]) == (9 - 8) + (8 - 4) and len(p1["prefix_slots"]) == 8 + 4
    b1 = s.seq_info(p1["seq_ids"][0])["blocks"]
    assert b1[:2] == blocks0[:2]
    assert p1["prefix_slots"][:8] == [blocks0[0] * bs + i for i in range(4)] + [blocks0[1] * bs + i for i in range(4)]
    free_before = s.num_free_blocks
    # everybody finishes: hashed blocks stay cached and count as free
    for sid in list(p0["seq_ids"]) + list(p1["seq_ids"]):
        s.finish(sid)
    assert s.num_cached_blocks == 2 and s.num_free_blocks == 24 and free_before < 24
    # a new request with the same chain still hits although nobody held the blocks in between
    s.add_group(3, 12, 1, 4, [], [11, 12, 13])
    p3 = s.plan_prefill()
    assert p3["cached_lens"] == [8] and s.seq_info(p3["seq_ids"][0])["blocks"][:2] == blocks0[:2]
    s.finish(p3["seq_ids"][0])
    assert s.num_cached_blocks == 3  # block 13 was registered by the call that followed its prefill plan
    # exhaust the plain free blocks: cached blocks are evicted (oldest release first) and their hashes forgotten
    s.add_group(4, 4 * 15, 1, 4, [], [])
    p4 = s.plan_prefill()
    assert p4["group_ids"] == [4]
    s.add_group(5, 9, 1, 2, [], [11, 12])
    p5 = s.plan_prefill()
    assert p5["group_ids"] == [5] and p5["cached_lens"][0] in (0, 4, 8)
    s.finish(p4["seq_ids"][0])
    s.finish(p5["seq_ids"][0])
    s.clear_prefix_cache()
    assert s.num_cached_blocks == 0 and s.num_free_blocks == 24
    s.add_group(6, 9, 1, 2, [], [11, 12])
    assert s.plan_prefill()["cached_lens"] == [0]


def test_prefix_cache_randomised_invariants():
    """Random add / prefill / decode / finish / clear sequences with prompts drawn from a few shared chains. After every
    operation: blocks of live sequences are distinct unless they are shared prompt blocks of the same chain, the number
    of free blocks plus the blocks held by live sequences equals the pool, slot mappings never point into a cached
    prefix, and at the end everything is free again."""
    rng = np.random.default_rng(7)
    bs, nb = 4, 96
    s = _sched(num_blocks=nb, block_size=bs, max_seqs=12, max_blocks_per_seq=24, max_prefill_tokens=256)
    chains = [[int(h) for h in rng.integers(1, 1 << 60, 8)] for _ in range(3)]  # hash chains of 3 "system prompts"
    live = {}   # seq_id -> group id
    gid = 0
    group_chain = {}
    hit_tokens = 0
    for it in range(400):
        op = rng.integers(0, 10)
        if op < 3 and s.num_waiting < 4:
            c = int(rng.integers(0, 3))
            full = int(rng.integers(0, 8))
            plen = full * bs + int(rng.integers(0, bs)) or 1
            hashes = chains[c][:plen // bs] if rng.random() < 0.8 else []
            s.add_group(gid, plen, int(rng.integers(1, 4)), int(rng.integers(1, 12)), [], hashes)
            group_chain[gid] = (c, hashes)
            gid += 1
        elif op < 5:
            p = s.plan_prefill()
            assert len(p["cached_lens"]) == len(p["group_ids"])
            assert sum(p["prompt_lens"]) - sum(p["cached_lens"]) == len(p["slot_mapping"])
            assert sum(p["cached_lens"]) == len(p["prefix_slots"])
            assert not (set(p["slot_mapping"]) & set(p["prefix_slots"]))
            hit_tokens += sum(p["cached_lens"])
            for g, c, L in zip(p["group_ids"], p["cached_lens"], p["prompt_lens"]):
                assert c % bs == 0 and c < L and c <= len(group_chain[g][1]) * bs
            for sid in p["seq_ids"]:
                live[sid] = s.seq_info(sid)["group_id"]
        elif op < 8:
            d = s.plan_decode()
            for sid in d["preempted"]:
                live.pop(sid, None)
                s.finish(sid)
            # sequences reaching their length limit finish
            for sid in list(live):
                info = s.seq_info(sid)
                if info is not None and info["len"] >= info["max_len"]:
                    s.finish(sid)
                    live.pop(sid)
        elif op < 9 and live:
            sid = list(live)[int(rng.integers(0, len(live)))]
            s.finish(sid)
            live.pop(sid)
        else:
            if rng.random() < 0.2:
                s.clear_prefix_cache()
        # ---- invariants ----
        held = {}
        for sid in live:
            info = s.seq_info(sid)
            assert info is not None
            for b in info["blocks"]:
                held.setdefault(b, []).append(sid)
        for b, owners in held.items():
            if len(owners) > 1:  # shared blocks: prompt blocks of the same group, or of groups on the same chain
                cs = {group_chain[live[o]][0] for o in owners}
                assert len(cs) == 1, (b, owners)
        assert s.num_free_blocks + len(held) == nb, (it, s.num_free_blocks, len(held))
        assert s.num_cached_blocks <= nb
    assert hit_tokens > 0, "the workload must produce prefix hits"
    for sid in list(live):
        s.finish(sid)
    assert s.num_free_blocks == nb and s.num_running == 0
    s.clear_prefix_cache()
    assert s.num_cached_blocks == 0 and s.num_free_blocks == nb
