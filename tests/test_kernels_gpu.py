"""Numerics of every sm_100a kernel against plain PyTorch fp32 references."""
import math

import pytest
import torch

from gpu_util import make_tiles, native, ref_attention, rel_err, status_word

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (1000, 1536, 1536), (333, 2048, 1536), (77, 200, 72),
                                   (4099, 1536, 1024), (64, 1536, 8960), (256, 17920, 1536)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_tcgen05(M, N, K, a_mn, b_mn):
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a row pitch that is a multiple of 8")
    C = native()
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    A = a.t() if a_mn else a
    B = b.t() if b_mn else b
    ref = A.float() @ B.float().t()
    d = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    st = status_word()
    C.gemm_bf16(a, b, d, a_mn, b_mn, None, 1.0, False, st, None)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert rel_err(d, ref) < 1e-2


def test_gemm_epilogues():
    C = native()
    torch.manual_seed(1)
    M, N, K = 512, 2048, 1536
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    st = status_word()
    d = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    C.gemm_bf16(a, b, d, False, False, bias, 1.0, False, st, res)
    ref = a.float() @ b.float().t() + bias.float() + res.float()
    assert rel_err(d, ref) < 1e-2
    # fp32 accumulate (weight-gradient path)
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    want = acc + a.float() @ b.float().t()
    C.gemm_bf16(a, b, acc, False, False, None, 1.0, True, st, None)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert rel_err(acc, want) < 1e-4


@pytest.mark.parametrize("lens,Hq,Hkv,D", [([128], 1, 1, 128), ([100], 2, 1, 128), ([300, 77, 513, 1], 12, 2, 128),
                                           ([1000, 250], 4, 2, 64), ([700, 333], 7, 1, 128), ([640, 129], 8, 1, 128)])
def test_attention_forward_backward(lens, Hq, Hkv, D):
    C = native()
    torch.manual_seed(0)
    T, Cc = sum(lens), (Hq + 2 * Hkv) * D
    qkv = torch.randn(T, Cc, device=DEV).to(torch.bfloat16)
    dout = torch.randn(T, Hq * D, device=DEV).to(torch.bfloat16)
    out = torch.zeros(T, Hq * D, device=DEV, dtype=torch.bfloat16)
    lse = torch.zeros(Hq, T, device=DEV)
    tiles = make_tiles(lens)
    st = status_word()
    sc = 1.0 / math.sqrt(D)
    C.attn_varlen_fwd(qkv, out, lse, tiles, Hq, Hkv, D, sc, st)
    x = qkv.float().clone().requires_grad_(True)
    ro, rl = ref_attention(x, lens, Hq, Hkv, D)
    ro.backward(dout.float())
    assert rel_err(out, ro.detach()) < 1.5e-2
    assert (lse - rl.detach()).abs().max().item() < 2e-2
    delta = torch.empty(Hq, T, device=DEV)
    dq_acc = torch.empty(T, Hq * D, device=DEV)
    dqkv = torch.zeros(T, Cc, device=DEV, dtype=torch.bfloat16)
    C.attn_varlen_bwd(qkv, out, dout, lse, delta, dq_acc, dqkv, tiles, Hq, Hkv, D, sc, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    for a0, a1 in ((0, Hq * D), (Hq * D, (Hq + Hkv) * D), ((Hq + Hkv) * D, Cc)):
        assert rel_err(dqkv[:, a0:a1], x.grad[:, a0:a1]) < 2e-2


def test_elementwise_ops():
    C = native()
    torch.manual_seed(0)
    T, H, F = 333, 1536, 4096
    x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    y = torch.empty_like(x)
    rstd = torch.empty(T, device=DEV)
    C.rmsnorm_fwd(x, w, y, rstd, 1e-6)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    assert rel_err(y, ref.detach()) < 1e-2
    dy = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    ref.backward(dy.float())
    dx = torch.empty_like(x)
    dw = torch.zeros(H, device=DEV)
    C.rmsnorm_bwd(dy, x, w, rstd, dx, dw, False)
    assert rel_err(dx, xf.grad) < 1.5e-2
    assert rel_err(dw, wf.grad) < 1.5e-2
    # swiglu
    gu = torch.randn(T, 2 * F, device=DEV).to(torch.bfloat16)
    guf = gu.float().requires_grad_(True)
    r = torch.nn.functional.silu(guf[:, :F]) * guf[:, F:]
    act = torch.empty(T, F, device=DEV, dtype=torch.bfloat16)
    C.swiglu_fwd(gu, act)
    assert rel_err(act, r.detach()) < 1e-2
    da = torch.randn(T, F, device=DEV).to(torch.bfloat16)
    r.backward(da.float())
    dgu = torch.empty_like(gu)
    C.swiglu_bwd(gu, da, dgu)
    assert rel_err(dgu, guf.grad) < 1.5e-2
    # rope forward then backward is the identity
    from async_grpo_nccl_b200.ops import reference as R

    D, heads = 128, 6
    cos_t, sin_t = R.rope_tables(D, 4096, 1e6, DEV)
    qkv = torch.randn(T, (heads + 2) * D, device=DEV).to(torch.bfloat16)
    pos = torch.randint(0, 4096, (T,), device=DEV, dtype=torch.int32)
    ref_rot = R.apply_rope(qkv[:, :heads * D].reshape(T, heads, D).float(), pos, cos_t, sin_t).reshape(T, heads * D)
    rot = qkv.clone()
    C.rope_inplace(rot, pos, cos_t, sin_t, heads, D, False)
    assert rel_err(rot[:, :heads * D], ref_rot) < 1e-2
    assert torch.equal(rot[:, heads * D:], qkv[:, heads * D:])
    C.rope_inplace(rot, pos, cos_t, sin_t, heads, D, True)
    assert rel_err(rot, qkv) < 2e-2
    # embedding + column sums
    V = 1000
    table = torch.randn(V, H, device=DEV).to(torch.bfloat16)
    ids = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    e = torch.empty(T, H, device=DEV, dtype=torch.bfloat16)
    C.embedding_fwd(ids, table, e)
    assert torch.equal(e, table[ids.long()])
    dt = torch.zeros(V, H, device=DEV)
    C.embedding_bwd(ids, dy, dt)
    want = torch.zeros(V, H, device=DEV).index_add_(0, ids.long(), dy.float())
    assert rel_err(dt, want) < 1e-3
    cs = torch.zeros(H, device=DEV)
    C.colsum(dy, cs)
    assert rel_err(cs, dy.float().sum(0)) < 1e-3


def test_adamw_and_norm():
    C = native()
    from async_grpo_nccl_b200.ops import reference as R

    torch.manual_seed(0)
    n = 1_000_003
    p = torch.randn(n, device=DEV)
    m = torch.randn(n, device=DEV) * 0.01
    v = torch.rand(n, device=DEV) * 0.01
    g = torch.randn(n, device=DEV)
    pr, mr, vr, gr = p.clone(), m.clone(), v.clone(), g.clone()
    ns = torch.zeros(1, device=DEV)
    C.sumsq(g, 1.0, ns)
    assert abs(ns.item() - g.double().pow(2).sum().item()) / g.double().pow(2).sum().item() < 1e-4
    p16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    C.adamw_step(p, m, v, g, p16, 1e-3, 0.9, 0.999, 1e-8, 0.01, 3, 1.0, ns, 1.0, True)
    R.adamw_step_(pr, mr, vr, gr, 1e-3, 0.9, 0.999, 1e-8, 0.01, 3, 1.0, 1.0, ns)
    assert rel_err(p, pr) < 1e-5 and rel_err(m, mr) < 1e-5 and rel_err(v, vr) < 1e-5
    assert torch.equal(p16, p.to(torch.bfloat16))
    assert float(g.abs().max()) == 0.0


@pytest.mark.parametrize("T,H,V,temp,beta", [(128, 256, 1024, 1.0, 0.0), (300, 256, 1000, 0.7, 0.001), (1000, 1536, 5000, 1.0, 0.0),
                                             (2048, 512, 18992, 1.3, 0.01)])
def test_lmhead_loss(T, H, V, temp, beta):
    C = native()
    from async_grpo_nccl_b200.ops import reference as R

    torch.manual_seed(0)
    h = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    W = (torch.randn(V, H, device=DEV) * 0.05).to(torch.bfloat16)
    labels = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    labels[torch.rand(T, device=DEV) < 0.2] = -100
    adv = torch.randn(T, device=DEV)
    hf, Wf = h.float().requires_grad_(True), W.float().requires_grad_(True)
    logp_ref, ent_ref = R.lmhead_logprob_entropy(hf, Wf, labels, temp)
    mask = labels >= 0
    old = (logp_ref.detach() + 0.3 * torch.randn(T, device=DEV)) * mask
    refl = (logp_ref.detach() + 0.1 * torch.randn(T, device=DEV)) * mask
    loss_sum, stats_ref = R.grpo_token_loss(logp_ref, old, refl, adv, labels, 0.2, 0.28, 3.0, beta, ent_ref)
    gw = 0.7 / max(1, int(mask.sum()))
    (loss_sum * gw).backward()
    st = status_word()
    groups = C.lmhead_num_groups(V, T)
    partials = torch.empty(3 * groups * T, device=DEV)
    ll = torch.zeros(T, device=DEV)
    logp, ent, lse = (torch.empty(T, device=DEV) for _ in range(3))
    C.lmhead_logprob(h, W, labels, temp, partials, ll, logp, ent, lse, st)
    ns = C.grpo_num_loss_stats()
    assert ns == len(R.LOSS_STAT_NAMES)
    dlogp, stats = torch.empty(T, device=DEV), torch.zeros(ns, device=DEV)
    C.grpo_token_loss(logp, old, refl if beta > 0 else None, adv, labels, ent, None, 0.2, 0.28, 3.0, beta, gw, dlogp, stats)
    dz = torch.empty(T, 1024, device=DEV, dtype=torch.bfloat16)
    dh, dW = torch.empty(T, H, device=DEV), torch.zeros(V, H, device=DEV)
    C.lmhead_backward(h, W, labels, lse, dlogp, temp, dz, dh, dW, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert (logp - logp_ref.detach()).abs().max().item() < 2e-2
    assert (ent - ent_ref).abs().max().item() < 2e-2
    assert abs(stats[1].item() - loss_sum.item()) < 2e-2 * max(1.0, abs(loss_sum.item()))
    for i in (0, 4, 5, 11, 12, 13):  # counts must agree up to tokens that sit on a clip boundary
        assert abs(stats[i].item() - stats_ref[i].item()) <= max(3.0, 0.01 * stats_ref[0].item())
    # (a) d loss / d logp, element by element, on tokens whose ratio is not next to a clip boundary (the kernel's own logp
    # differs from the fp32 one by bf16 noise, so a token within a few percent of a boundary may take the other branch)
    leaf = logp_ref.detach().clone().requires_grad_(True)
    loss2, _ = R.grpo_token_loss(leaf, old, refl, adv, labels, 0.2, 0.28, 3.0, beta, ent_ref.detach())
    (loss2 * gw).backward()
    ratio = torch.exp(logp_ref.detach() - old)
    far = mask.clone()
    for edge in (0.8, 1.28, 3.0):
        far &= (ratio - edge).abs() > 0.05 * edge
    assert far.float().mean().item() > 0.5
    err = (dlogp - leaf.grad)[far].abs()
    assert (err <= 0.05 * leaf.grad[far].abs() + 1e-7).all(), err.max().item()
    assert (dlogp[~mask] == 0).all()
    # (b) the lm_head backward itself, element by element: gradients of sum_t dlogp[t] * logp[t] for the kernel's dlogp
    h2, W2 = h.float().requires_grad_(True), W.float().requires_grad_(True)
    logp2, _ = R.lmhead_logprob_entropy(h2, W2, labels, temp)
    (logp2 * dlogp.detach() * mask).sum().backward()
    assert rel_err(dh, h2.grad) < 2e-2, rel_err(dh, h2.grad)
    assert rel_err(dW, W2.grad) < 2e-2, rel_err(dW, W2.grad)
    # and the end-to-end direction against the fp32 objective
    cos = torch.nn.functional.cosine_similarity
    assert cos(dh.flatten(), hf.grad.flatten(), dim=0).item() > 0.97
    assert cos(dW.flatten(), Wf.grad.flatten(), dim=0).item() > 0.97


def test_lmhead_full_vocabulary_tail_tile():
    """V = 151936 (1187 column tiles of 128, the last 256-wide tile half empty) with T = 4096: log-probabilities, entropy and
    both gradients against fp32 PyTorch computed in row chunks."""
    C = native()
    from async_grpo_nccl_b200.ops import reference as R

    torch.manual_seed(1)
    T, H, V, temp = 4096, 256, 151936, 1.0
    h = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    W = (torch.randn(V, H, device=DEV) * 0.05).to(torch.bfloat16)
    labels = torch.randint(0, V, (T,), device=DEV, dtype=torch.int32)
    labels[:64] = V - 1 - torch.arange(64, device=DEV, dtype=torch.int32)  # labels inside the tail tile
    labels[torch.rand(T, device=DEV) < 0.1] = -100
    mask = labels >= 0
    st = status_word()
    groups = C.lmhead_num_groups(V, T)
    partials = torch.empty(3 * groups * T, device=DEV)
    ll = torch.zeros(T, device=DEV)
    logp, ent, lse = (torch.empty(T, device=DEV) for _ in range(3))
    C.lmhead_logprob(h, W, labels, temp, partials, ll, logp, ent, lse, st)
    dlogp = torch.randn(T, device=DEV) * mask / T
    dz = torch.empty(T, 1024, device=DEV, dtype=torch.bfloat16)
    dh, dW = torch.empty(T, H, device=DEV), torch.zeros(V, H, device=DEV)
    C.lmhead_backward(h, W, labels, lse, dlogp, temp, dz, dh, dW, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    Wf = W.float().requires_grad_(True)
    dh_ref = torch.empty(T, H, device=DEV)
    for r0 in range(0, T, 512):  # fp32 reference in row chunks (a [512, V] fp32 block is 311 MB)
        hf = h[r0:r0 + 512].float().requires_grad_(True)
        lp, en = R.lmhead_logprob_entropy(hf, Wf, labels[r0:r0 + 512], temp)
        assert (logp[r0:r0 + 512] - lp.detach()).abs().max().item() < 2e-2
        assert (ent[r0:r0 + 512] - en.detach()).abs().max().item() < 2e-2
        (lp * dlogp[r0:r0 + 512] * mask[r0:r0 + 512]).sum().backward()
        dh_ref[r0:r0 + 512] = hf.grad
    assert rel_err(dh, dh_ref) < 2e-2
    assert rel_err(dW, Wf.grad) < 2e-2
    assert rel_err(dW[V - 256:], Wf.grad[V - 256:]) < 2e-2  # rows of the tail tile


def test_paged_decode_and_kv_write():
    C = native()
    torch.manual_seed(0)
    D, bs = 128, 16
    for (B, Hq, Hkv, lens, splits) in [(2, 12, 2, [1, 16], 1), (3, 12, 2, [100, 17, 1333], 4), (4, 28, 4, [5, 64, 65, 900], 3),
                                       (2, 8, 1, [2000, 31], 8), (3, 40, 8, [7, 300, 129], 2)]:
        max_blocks = (max(lens) + bs - 1) // bs
        nblk = sum((L + bs - 1) // bs for L in lens) + 3
        kc = torch.randn(nblk, Hkv, bs, D, device=DEV).to(torch.bfloat16)
        vc = torch.randn(nblk, Hkv, bs, D, device=DEV).to(torch.bfloat16)
        perm = torch.randperm(nblk).tolist()
        bt = torch.zeros(B, max_blocks, dtype=torch.int32)
        pi = 0
        for b, L in enumerate(lens):
            for j in range((L + bs - 1) // bs):
                bt[b, j] = perm[pi]
                pi += 1
        bt = bt.to(DEV)
        sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
        qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=DEV).to(torch.bfloat16)
        out = torch.zeros(B, Hq * D, device=DEV, dtype=torch.bfloat16)
        po = torch.empty(B * Hkv * splits * 8 * D, device=DEV)
        pml = torch.empty(B * Hkv * splits * 16, device=DEV)
        st = status_word()
        # the newest token's K/V goes into the cache first (decode order)
        C.kv_cache_write_decode(qkv, bt, sl, kc, vc, Hq, Hkv, D, st)
        C.paged_decode_attn(qkv, kc, vc, bt, sl, out, Hq, Hkv, D, 1 / math.sqrt(D), splits, po, pml, st)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        G = Hq // Hkv
        ref = torch.zeros(B, Hq, D, device=DEV)
        for b, L in enumerate(lens):
            nb = (L + bs - 1) // bs
            k = kc[bt[b, :nb].long()].permute(1, 0, 2, 3).reshape(Hkv, nb * bs, D)[:, :L].float()
            v = vc[bt[b, :nb].long()].permute(1, 0, 2, 3).reshape(Hkv, nb * bs, D)[:, :L].float()
            assert torch.equal(k[:, L - 1].to(torch.bfloat16).reshape(-1), qkv[b, Hq * D:(Hq + Hkv) * D])
            q = qkv[b, :Hq * D].view(Hkv, G, D).float()
            s = torch.einsum("hgd,hld->hgl", q, k) / math.sqrt(D)
            ref[b] = torch.einsum("hgl,hld->hgd", torch.softmax(s, -1), v).reshape(Hq, D)
        assert rel_err(out.view(B, Hq, D), ref) < 1.5e-2
        # split-KV merge done by the last split CTA (arrival tickets) instead of a second kernel: same result, and the
        # counters are back at zero so that the next launch (second call) starts clean
        tickets = torch.zeros(B * Hkv, device=DEV, dtype=torch.int32)
        for _ in range(2):
            out2 = torch.zeros_like(out)
            C.paged_decode_attn(qkv, kc, vc, bt, sl, out2, Hq, Hkv, D, 1 / math.sqrt(D), splits, po, pml, st, tickets)
            torch.cuda.synchronize()
            assert torch.equal(out2, out)
            assert int(tickets.abs().max()) == 0 and int(st.item()) == 0


def test_lm_sample_greedy_and_distribution():
    C = native()
    torch.manual_seed(0)
    R_, H, V = 64, 256, 5000
    h = torch.randn(R_, H, device=DEV).to(torch.bfloat16)
    W = (torch.randn(V, H, device=DEV) * 0.2).to(torch.bfloat16)
    st = status_word()
    groups = C.lm_sample_num_groups(V, R_)
    pf = torch.empty(4 * groups * R_, device=DEV)
    pi = torch.empty(groups * R_, device=DEV, dtype=torch.int32)
    tok = torch.empty(R_, device=DEV, dtype=torch.int32)
    lp = torch.empty(R_, device=DEV)
    seeds = torch.arange(R_, device=DEV, dtype=torch.int64) * 7919 + 13
    C.lm_sample(h, W, 0.0, seeds, pf, pi, tok, lp, st)
    z = h.float() @ W.float().t()
    top2 = z.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.05
    assert torch.equal(tok.long()[clear], z.argmax(-1)[clear])
    ref_lp = torch.log_softmax(z, -1).gather(1, tok.long()[:, None])[:, 0]
    assert (lp - ref_lp).abs().max().item() < 2e-2
    # sampling frequencies follow softmax(z / temperature)
    R2, V2 = 4096, 512
    h1 = torch.randn(1, H, device=DEV).to(torch.bfloat16).expand(R2, H).contiguous()
    W2 = (torch.randn(V2, H, device=DEV) * 0.1).to(torch.bfloat16)
    groups = C.lm_sample_num_groups(V2, R2)
    pf = torch.empty(4 * groups * R2, device=DEV)
    pi = torch.empty(groups * R2, device=DEV, dtype=torch.int32)
    tok = torch.empty(R2, device=DEV, dtype=torch.int32)
    counts = torch.zeros(V2, device=DEV)
    for r in range(16):
        seeds = torch.arange(R2, device=DEV, dtype=torch.int64) + r * 1000003 + 17
        C.lm_sample(h1, W2, 0.8, seeds, pf, pi, tok, None, st)
        counts += torch.bincount(tok.long(), minlength=V2).float()
    p = torch.softmax((h1[0].float() @ W2.float().t()) / 0.8, -1)
    tv = 0.5 * (counts / counts.sum() - p).abs().sum().item()
    assert tv < 0.05
    assert int(st.item()) == 0
    # same seeds -> same tokens
    t2 = torch.empty_like(tok)
    C.lm_sample(h1, W2, 0.8, seeds, pf, pi, t2, None, st)
    assert torch.equal(t2, tok)


def test_bounded_wait_reports_status_instead_of_hanging():
    """A flag that nobody sets: the waiting kernel gives up after its budget and returns an error status."""
    C = native()
    flag = torch.zeros(1, device=DEV, dtype=torch.int64)
    st = status_word()
    C.wait_flag_probe(flag, 1, 0.05, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 5  # kStatusPeerFlagTimeout
    flag.fill_(3)
    st.zero_()
    C.wait_flag_probe(flag, 2, 0.05, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0


@pytest.mark.parametrize("M", [1, 64, 128, 200, 256])
@pytest.mark.parametrize("N,K", [(1536, 1536), (2048, 1536), (1536, 8960), (200, 520), (17920, 1536)])
def test_gemm_skinny_cluster_split_k(M, N, K):
    """Decode-time shapes take the cluster split-K kernel (reduction through distributed shared memory)."""
    C = native()
    torch.manual_seed(M * 7 + N)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    d = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    st = status_word()
    C.gemm_bf16(a, b, d, False, False, bias, 1.0, False, st, res)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = a.float() @ b.float().t() + bias.float() + res.float()
    assert rel_err(d, ref) < 1e-2


# ---- fused compute + collective kernels, owners emulated by separate buffers of one GPU (one launch: no kernel waits
# on another launch). The 2-GPU test in test_multi_gpu.py runs the same kernels over real peer memory. ----
@pytest.mark.parametrize("W,b_mn", [(1, False), (4, False), (2, True)])
def test_ag_gemm_emulated_owners(W, b_mn):
    C = native()
    torch.manual_seed(3)
    M, N, K = 1024, 2048, 1536
    rel = 1536 * 3  # B starts after some other parameters of the unit
    n_unit = ((rel + N * K + 4096 + 128 * W - 1) // (128 * W)) * (128 * W)
    n_per = n_unit // W
    unit = torch.randn(n_unit, device=DEV, dtype=torch.bfloat16)
    shards = [unit[r * n_per:(r + 1) * n_per].clone() for r in range(W)]
    staging = torch.zeros(n_unit, device=DEV, dtype=torch.bfloat16)
    chunk = 65536
    flags = torch.zeros((n_unit + chunk - 1) // chunk, device=DEV, dtype=torch.int64)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    bshape = (K, N) if b_mn else (N, K)
    b = staging[rel:rel + N * K].view(bshape)
    d = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    st = status_word()
    C.ag_gemm(a, b, d, False, b_mn, None, False, st, None, src_ptrs=[s.data_ptr() for s in shards], my_rank=0,
              staging=staging, n_per_owner=n_per, flags=flags, epoch=1, chunk_elems=chunk, n_copy=8)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(staging, unit)
    assert bool((flags == 1).all())
    Bm = unit[rel:rel + N * K].view(bshape).float()
    ref = a.float() @ (Bm if b_mn else Bm.t())
    assert rel_err(d, ref) < 1e-2
    # prefetch mode: B is elsewhere, the launch gathers a second unit for later launches
    unit2 = torch.randn(n_unit, device=DEV, dtype=torch.bfloat16)
    shards2 = [unit2[r * n_per:(r + 1) * n_per].clone() for r in range(W)]
    staging2 = torch.zeros_like(staging)
    flags2 = torch.zeros_like(flags)
    b2 = Bm.to(torch.bfloat16).contiguous()
    d2 = torch.empty_like(d)
    C.ag_gemm(a, b2, d2, False, b_mn, None, False, st, None, src_ptrs=[s.data_ptr() for s in shards2], my_rank=0,
              staging=staging2, n_per_owner=n_per, flags=flags2, epoch=7, chunk_elems=chunk, n_copy=16)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(staging2, unit2) and bool((flags2 == 7).all())
    assert torch.equal(d2, d)
    # the gather alone
    staging3 = torch.zeros_like(staging)
    C.unit_gather([s.data_ptr() for s in shards2], 0, staging3, n_per, flags2, 8, chunk, 32)
    torch.cuda.synchronize()
    assert torch.equal(staging3, unit2) and bool((flags2 == 8).all())


@pytest.mark.parametrize("W", [1, 4])
def test_gemm_reduce_scatter_emulated_owners(W):
    C = native()
    torch.manual_seed(4)
    T, No, Ki = 2048, 1536, 1024       # dW[No, Ki] = dy[T, No]^T . x[T, Ki]
    rel = 1536 + 128
    n_unit = ((rel + No * Ki + 1000 + 128 * W - 1) // (128 * W)) * (128 * W)
    n_per = n_unit // W
    dy = torch.randn(T, No, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(T, Ki, device=DEV, dtype=torch.bfloat16)
    before = torch.randn(n_unit, device=DEV, dtype=torch.float32)
    shards = [before[r * n_per:(r + 1) * n_per].clone() for r in range(W)]
    st = status_word()
    C.gemm_rs(dy, x, True, True, 0.5, [s.data_ptr() for s in shards], n_per, rel, Ki, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    got = torch.cat(shards)
    want = before.clone()
    want[rel:rel + No * Ki] += 0.5 * (dy.float().t() @ x.float()).reshape(-1)
    assert rel_err(got, want) < 1e-4
    # small vectors and the embedding group take the elementwise scatter
    src = torch.randn(5000, device=DEV, dtype=torch.float32)
    src[100:400] = 0
    keep = src.clone()
    C.scatter_add_f32(src, 128, [s.data_ptr() for s in shards], n_per, True)
    torch.cuda.synchronize()
    want[128:128 + 5000] += keep
    assert rel_err(torch.cat(shards), want) < 1e-4
    assert float(src.abs().max()) == 0.0


@pytest.mark.parametrize("M,H,F", [(64, 1536, 8960), (128, 512, 1408), (200, 1536, 8960)])
def test_decode_fused_gemms_match_unfused_layer_math(M, H, F):
    """Folded-norm split-K GEMM (row scale in, row sum of squares out) and the gate/up + SwiGLU GEMM against the plain
    sequence rmsnorm -> linear -> swiglu in fp32."""
    C = native()
    torch.manual_seed(7)
    x = torch.randn(M, H, device=DEV, dtype=torch.bfloat16) * 3
    ln = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)
    wq = (torch.randn(2048, H, device=DEV) * 0.03).to(torch.bfloat16)
    wgu = (torch.randn(2 * F, H, device=DEV) * 0.03).to(torch.bfloat16)
    bias = torch.randn(2048, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, H, device=DEV, dtype=torch.bfloat16)
    wd = (torch.randn(H, F, device=DEV) * 0.03).to(torch.bfloat16)
    eps = 1e-6
    st = status_word()
    fq, fgu = torch.empty_like(wq), torch.empty_like(wgu)
    C.fold_norm_weight(wq, ln, fq)
    C.fold_norm_weight(wgu, ln, fgu)
    assert rel_err(fq, wq.float() * ln.float()) < 5e-3
    xf = x.float()
    ss = (xf * xf).sum(-1)
    hn = xf * torch.rsqrt(ss / H + eps)[:, None] * ln.float()
    # qkv-style GEMM with folded norm and bias
    qkv = torch.empty(M, 2048, device=DEV, dtype=torch.bfloat16)
    ssf = (ss.double() * 2 ** 30).round().to(torch.int64)  # the kernels exchange the statistic in fixed point
    assert C.gemm_decode(x, fq, qkv, bias, None, ssf, None, eps, st)
    assert rel_err(qkv, hn @ wq.float().t() + bias.float()) < 1.5e-2
    # gate/up + swiglu with folded norm
    act = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    C.gemm_swiglu(x, fgu, act, ssf, eps, st)
    gu = hn @ wgu.float().t()
    ref_act = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    assert rel_err(act, ref_act) < 2e-2
    # down-style GEMM with residual and sum-of-squares output
    out = torch.empty(M, H, device=DEV, dtype=torch.bfloat16)
    ss_out = torch.zeros(M, device=DEV, dtype=torch.int64)
    assert C.gemm_decode(act, wd, out, None, res, None, ss_out, eps, st)
    ref_out = act.float() @ wd.float().t() + res.float()
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert rel_err(out, ref_out) < 1e-2
    assert rel_err(ss_out.double() / 2 ** 30, (ref_out * ref_out).sum(-1)) < 1e-2
    # embedding lookup with the statistic
    table = torch.randn(1000, H, device=DEV, dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (M,), device=DEV, dtype=torch.int32)
    ssb = torch.full((5, 256), 7, device=DEV, dtype=torch.int64)
    xo = torch.empty(M, H, device=DEV, dtype=torch.bfloat16)
    C.embedding_sumsq(ids, table, xo, ssb)
    assert torch.equal(xo, table[ids.long()])
    assert rel_err(ssb[0, :M].double() / 2 ** 30, (xo.float() ** 2).sum(-1)) < 1e-5
    assert int(ssb[1:, :M].abs().max()) == 0 and int(ssb[1:, M:].min()) == 7


@pytest.mark.parametrize("M,Hq,Hkv,H", [(32, 12, 2, 1536), (100, 4, 2, 512), (128, 12, 2, 1536)])
def test_qkv_gemm_with_rope_and_cache_write_epilogue(M, Hq, Hkv, H):
    """The fused decode qkv projection (folded-norm scale, bias, RoPE, paged KV write in the GEMM epilogue) against
    the two-kernel sequence gemm_decode -> rope_kv_write_decode."""
    C = native()
    torch.manual_seed(11)
    D, bs, nblk = 128, 16, 64 + M
    N = (Hq + 2 * Hkv) * D
    x = torch.randn(M, H, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(N, H, device=DEV) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    ss = ((x.double() ** 2).sum(-1) * 2 ** 30).round().to(torch.int64)
    max_pos = 512
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=DEV).float() / D))
    ang = torch.arange(max_pos, device=DEV).float()[:, None] * inv[None, :]
    cos_t, sin_t = ang.cos().contiguous(), ang.sin().contiguous()
    lens = torch.randint(1, 300, (M,), device=DEV, dtype=torch.int32)
    lens[0] = 0  # an idle row: rotated at position 0, nothing written to the cache
    max_blocks = 32
    perm = torch.randperm(nblk, device=DEV)[:M].to(torch.int32)
    bt = torch.full((M, max_blocks), -1, device=DEV, dtype=torch.int32)
    for r in range(M):
        L = int(lens[r])
        if L > 0:
            bt[r, (L - 1) // bs] = perm[r]
    st = status_word()
    outs = []
    for fused in (False, True):
        kc = torch.zeros(nblk, Hkv, bs, D, device=DEV, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        qkv = torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
        if fused:
            assert C.gemm_decode_rope(x, w, qkv, bias, ss, 1e-6, cos_t, sin_t, bt, lens, kc, vc, Hq, Hkv, st)
        else:
            assert C.gemm_decode(x, w, qkv, bias, None, ss, None, 1e-6, st)
            C.rope_kv_write_decode(qkv, cos_t, sin_t, bt, lens, kc, vc, Hq, Hkv, D, st)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        outs.append((qkv, kc, vc))
    (q0, k0, v0), (q1, k1, v1) = outs
    assert rel_err(q1, q0.float()) < 1e-2
    assert rel_err(k1, k0.float()) < 1e-2 and rel_err(v1, v0.float()) < 1e-2
    # the same cache cells are written (and only those)
    assert torch.equal(k1.abs().sum(-1) > 0, k0.abs().sum(-1) > 0)
    assert torch.equal(v1.abs().sum(-1) > 0, v0.abs().sum(-1) > 0)


def test_peer_kernels_return_untouched_when_the_group_status_is_set():
    """A barrier that ran out of time leaves an error code in the group's status word; the kernels queued behind it
    (weight push, gradient pull, AdamW + publish) must then leave parameters, moments and destinations as they were."""
    C = native()
    torch.manual_seed(3)
    n = 4096
    st = status_word()
    src = torch.randn(n, device=DEV, dtype=torch.float32)
    dst = torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    p, m, v = src.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    g = torch.randn(n, device=DEV)
    partials = torch.ones(1, device=DEV)
    out, norm = torch.zeros(n, device=DEV), torch.zeros(1, device=DEV)
    try:
        C.set_comm_guard(st)
        st.fill_(7)  # what a timed-out barrier records
        C.weight_push(src, 0, 0, n, [dst.data_ptr()])
        C.adamw_push(p, m, v, g.clone(), 0, 0, n, 1e-2, 0.9, 0.999, 1e-8, 0.0, 1, 1.0, partials, 1.0, [dst.data_ptr()])
        C.rs_pull_sumsq([g.data_ptr()], 0, 0, 0, n, out, norm)
        torch.cuda.synchronize()
        assert dst.abs().sum().item() == 0 and torch.equal(p, src) and m.abs().sum().item() == 0 and v.abs().sum().item() == 0
        assert out.abs().sum().item() == 0 and norm.item() == 0
        st.zero_()
        C.weight_push(src, 0, 0, n, [dst.data_ptr()])
        C.rs_pull_sumsq([g.data_ptr()], 0, 0, 0, n, out, norm)
        torch.cuda.synchronize()
        assert torch.equal(dst, src.to(torch.bfloat16)) and torch.equal(out, g)
    finally:
        C.set_comm_guard(None)


def test_prefill_kv_write_reports_out_of_range_slots_and_skips_them():
    """A slot beyond the cache is reported through the status word and not written (index checks never fault)."""
    C = native()
    torch.manual_seed(5)
    Hq, Hkv, D, bs, nblk, T = 4, 2, 128, 16, 8, 6
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV).to(torch.bfloat16)
    kc = torch.zeros(nblk, Hkv, bs, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.tensor([0, 17, -1, nblk * bs - 1, nblk * bs, nblk * bs + 1000], device=DEV, dtype=torch.int32)
    st = status_word()
    C.kv_cache_write(qkv, slots, kc, vc, Hq, Hkv, D, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 6  # bad index
    written = (kc.abs().sum(-1) > 0).sum().item()
    assert written == 3 * Hkv
    k_rows = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    assert torch.equal(kc[0, :, 0], k_rows[0]) and torch.equal(kc[1, :, 1], k_rows[1]) and torch.equal(kc[nblk - 1, :, bs - 1], k_rows[3])
