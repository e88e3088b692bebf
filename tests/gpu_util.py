"""Shared helpers for the GPU kernel tests: every kernel is compared with a plain PyTorch fp32 restatement."""
import math

import torch


def native():
    from async_grpo_nccl_b200.ops import native as _n

    return _n()


def make_tiles(lens, device="cuda"):
    tiles, start = [], 0
    for L in lens:
        for q0 in range(0, L, 128):
            tiles.append((start, L, q0, 0))
        start += L
    tiles.sort(key=lambda t: -t[2])
    return torch.tensor(tiles, dtype=torch.int32, device=device)


def ref_attention(qkv, lens, Hq, Hkv, D):
    T = qkv.shape[0]
    q = qkv[:, :Hq * D].reshape(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    g = Hq // Hkv
    outs, lses, s0 = [], [], 0
    for L in lens:
        qs = q[s0:s0 + L].transpose(0, 1)
        ks = k[s0:s0 + L].transpose(0, 1).repeat_interleave(g, 0)
        vs = v[s0:s0 + L].transpose(0, 1).repeat_interleave(g, 0)
        sc = qs @ ks.transpose(1, 2) / math.sqrt(D)
        mask = torch.ones(L, L, device=qkv.device, dtype=torch.bool).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        lses.append(torch.logsumexp(sc, -1))
        outs.append((torch.softmax(sc, -1) @ vs).transpose(0, 1).reshape(L, Hq * D))
        s0 += L
    return torch.cat(outs, 0), torch.cat(lses, 1)


def status_word():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def rel_err(a, b):
    return (a.float() - b.float()).abs().max().item() / max(1e-6, b.float().abs().max().item())
