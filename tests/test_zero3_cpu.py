"""Host-side logic of the fully sharded mode (parallel/zero3.py) against a recording stand-in for the extension:
which unit is gathered when, which gather rides on which GEMM, what the scatter sink sends where."""
import torch

from async_grpo_nccl_b200.models.config import PRESETS
from async_grpo_nccl_b200.models.layout import ParamLayout
from async_grpo_nccl_b200.parallel.zero3 import ScatterSink, ShardedWeights


class FakeNative:
    def __init__(self):
        self.calls = []

    def unit_gather(self, src_ptrs, my_rank, staging, n_per_owner, flags, epoch, chunk, n_ctas, status=None):
        self.calls.append(("unit_gather", tuple(src_ptrs), n_per_owner, epoch))

    def ag_gemm(self, a, b, out, a_mn, b_mn, bias, accumulate, status, residual, **kw):
        self.calls.append(("ag_gemm", tuple(kw["src_ptrs"]), kw["n_per_owner"], kw["epoch"], kw["n_copy"]))

    def gemm_bf16(self, *a):
        self.calls.append(("gemm_bf16",))

    def gemm_rs(self, dy, x, a_mn, b_mn, alpha, dst_ptrs, n_per_owner, unit_rel, ldd, status):
        self.calls.append(("gemm_rs", tuple(dst_ptrs), n_per_owner, unit_rel, ldd))

    def scatter_add_f32(self, src, unit_rel, dst_ptrs, n_per_owner, zero_src):
        self.calls.append(("scatter_add_f32", src.numel(), unit_rel, tuple(dst_ptrs), n_per_owner, zero_src))


def _layout(world=2):
    return ParamLayout(PRESETS["tiny128"], shard_world=world)


def test_gather_schedule_and_prefetch_rides_on_the_large_gemm():
    L, C = _layout(2), FakeNative()
    base = [1 << 20, 1 << 30]
    w = ShardedWeights(L, C, torch.device("cpu"), 0, base, n_copy=4, chunk_elems=4096)
    cfg = L.cfg
    # forward of layer 0: embedding group and unit 1 are gathered on their own, unit 2 is announced as next
    assert w.enter(0, None) == 1 and w.enter(1, 2) == 1
    assert [c[0] for c in C.calls] == ["unit_gather", "unit_gather"]
    lo1 = L.local_to_global_ranges(0)[1][0]
    assert C.calls[1][1] == tuple(b + 2 * lo1 for b in base)           # every owner's slice of unit 1, in bytes
    assert C.calls[1][2] == (L.unit_ranges[1][1] - L.unit_ranges[1][0]) // 2
    a = torch.zeros(2048, cfg.hidden_size)
    small = torch.zeros(cfg.qkv_dim, cfg.hidden_size)                    # qkv projection: too small to carry the copy
    big = torch.zeros(2 * cfg.intermediate_size, cfg.hidden_size)         # gate/up projection
    assert not w.wants_ride(a, small) and w.wants_ride(a, big)
    assert not w.wants_ride(torch.zeros(64, cfg.hidden_size), big)        # a decode-sized GEMM never carries a gather
    w.gemm_with_prefetch(a, big, None, False, False, None, False, None, None)
    assert C.calls[-1][0] == "ag_gemm" and C.calls[-1][4] == 4 and w.pending is None
    # unit 2 is now staged: entering it launches nothing; views of both layers resolve, epochs only ever grow
    assert w.enter(2, None) == 0
    assert w.view("layers.1.wqkv").shape == (cfg.qkv_dim, cfg.hidden_size)
    assert w.view("layers.0.wd").shape == (cfg.hidden_size, cfg.intermediate_size)
    epochs = [c[3] for c in C.calls]
    assert epochs == sorted(epochs) and len(set(epochs)) == len(epochs)
    # an optimizer step invalidates everything that is staged
    w.invalidate()
    assert not w.is_resident(0) and not w.is_resident(2)
    try:
        w.view("embed")
        raise AssertionError("a stale unit must not be readable")
    except RuntimeError:
        pass
    assert w.enter(0, None) == 1


def test_scatter_sink_routes_gradients_to_owner_shards():
    L, C = _layout(4), FakeNative()
    base = [0x1000_0000 * (r + 1) for r in range(4)]
    sink = ScatterSink(L, C, torch.device("cpu"), 1, base)
    cfg = L.cfg
    seg = L.segments["layers.1.wgu"]
    lo2 = L.local_to_global_ranges(1)[2][0]
    sink.wgrad(torch.zeros(8, 8), torch.zeros(8, 8), "layers.1.wgu", None)
    name, dst, n_per, rel, ldd = C.calls[-1]
    assert name == "gemm_rs" and dst == tuple(b + 4 * lo2 for b in base)
    assert n_per == (L.unit_ranges[2][1] - L.unit_ranges[2][0]) // 4
    assert rel == seg.offset - L.unit_ranges[2][0] and ldd == cfg.hidden_size
    # the embedding group accumulates locally (sparse row updates) and is sent once per microbatch
    sink.wgrad(torch.zeros(8, 8), torch.zeros(8, 8), "embed", None)
    assert C.calls[-1] == ("gemm_bf16",)
    assert sink.view("final_norm").numel() == cfg.hidden_size
    # small per-layer vectors share scratch that is sent and cleared when the layer's backward ends
    v = sink.view("layers.0.ln1")
    v += 1.0
    n_before = len(C.calls)
    sink.unit_done(1)
    sent = C.calls[n_before:]
    assert [c[0] for c in sent] == ["scatter_add_f32"] * len(sink.small_off)
    assert all(c[5] for c in sent)                                        # sources are zeroed by the kernel
    rels = {c[2] for c in sent}
    assert L.segments["layers.0.ln1"].offset - L.unit_ranges[1][0] in rels
    try:
        sink.view("layers.0.wqkv")
        raise AssertionError("large weight gradients have no local buffer")
    except RuntimeError:
        pass
    sink.unit_done(0)
    assert C.calls[-1][0] == "scatter_add_f32" and C.calls[-1][1] == L.unit_ranges[0][1] - L.unit_ranges[0][0]
