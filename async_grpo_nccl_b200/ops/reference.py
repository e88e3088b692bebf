"""Plain-PyTorch oracle of every op (fp32 math, differentiable through autograd).

It is what the CPU plumbing configuration runs and what every sm_100a kernel is tested against. The
loss follows what the reference's code computes (grpo_loss.py:146-250, 323-348): per-token
logprob = gathered logit - logsumexp on temperature-scaled logits, entropy = lse - sum(p * z), the
dual-clip objective with a token mean over unmasked positions, plus an optional k3 KL term against
supplied reference logprobs (weight ``kl_beta``; zero reproduces the reference objective).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

LOSS_STAT_NAMES = (
    "count", "loss_sum", "abs_log_ratio", "approx_kl", "clip_upper", "clip_lower", "log_ratio", "log_ratio_sq",
    "entropy", "adv", "adv_sq", "adv_pos", "adv_zero", "pg_clip", "old_entropy", "kl_ref", "logp", "dual_clip",
)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype)


def rope_tables(head_dim: int, max_pos: int, theta: float, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def apply_rope(x: torch.Tensor, pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, D]; rotate-half convention (first half pairs with second half)."""
    half = x.shape[-1] // 2
    c = cos_t[pos.long()][:, None, :]
    s = sin_t[pos.long()][:, None, :]
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: Sequence[int]) -> torch.Tensor:
    """Causal attention over packed segments. q: [T, Hq, D], k/v: [T, Hkv, D] -> [T, Hq, D] (GQA without repeat in memory)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    outs: List[torch.Tensor] = []
    scale = 1.0 / math.sqrt(D)
    for i in range(len(cu_seqlens) - 1):
        s, e = int(cu_seqlens[i]), int(cu_seqlens[i + 1])
        L = e - s
        if L == 0:
            continue
        qs = q[s:e].float().transpose(0, 1).reshape(Hkv, g, L, D)
        ks = k[s:e].float().transpose(0, 1)[:, None]
        vs = v[s:e].float().transpose(0, 1)[:, None]
        sc = torch.matmul(qs, ks.transpose(-1, -2)) * scale
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        o = torch.matmul(torch.softmax(sc, dim=-1), vs)  # [Hkv, g, L, D]
        outs.append(o.reshape(Hq, L, D).transpose(0, 1))
    if not outs:
        return torch.zeros_like(q)
    return torch.cat(outs, dim=0).to(q.dtype)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    f = gu.shape[-1] // 2
    g, u = gu[..., :f].float(), gu[..., f:].float()
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


def lmhead_logprob_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, temperature: float,
                           chunk: int = 4096, want_entropy: bool = True
                           ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """labels[t] is the (already shifted) target of row t, negative = masked. Returns fp32 [T] logprob (0 on
    masked rows) and entropy. Rows are processed in chunks so [T, V] never exists at once."""
    T = hidden.shape[0]
    lp_parts, ent_parts = [], []
    wf = weight.float()
    for s in range(0, T, chunk):
        z = hidden[s:s + chunk].float() @ wf.t() / temperature
        lse = torch.logsumexp(z, dim=-1)
        lab = labels[s:s + chunk]
        mask = lab >= 0
        gathered = z.gather(1, lab.clamp(min=0).long()[:, None])[:, 0]
        lp_parts.append(torch.where(mask, gathered - lse, torch.zeros_like(lse)))
        if want_entropy:
            with torch.no_grad():
                p = torch.softmax(z, dim=-1)
                ent_parts.append(lse.detach() - (p * z).sum(-1))
    logp = torch.cat(lp_parts) if lp_parts else hidden.new_zeros(0, dtype=torch.float32)
    ent = (torch.cat(ent_parts) if ent_parts else hidden.new_zeros(0, dtype=torch.float32)) if want_entropy else None
    return logp, ent


def grpo_token_loss(logp: torch.Tensor, old_logp: Optional[torch.Tensor], ref_logp: Optional[torch.Tensor],
                    adv: torch.Tensor, labels: torch.Tensor, clip_low: float, clip_high: float, clip_c: float,
                    kl_beta: float = 0.0, entropy: Optional[torch.Tensor] = None,
                    old_entropy: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (sum over valid tokens of the per-token objective, stats vector of sums in LOSS_STAT_NAMES order)."""
    mask = labels >= 0
    if old_logp is None:
        old_logp = logp.detach()
    lr = logp - old_logp
    ratio = torch.exp(lr)
    lower, upper = 1.0 - clip_low, 1.0 + clip_high
    unclipped = -adv * ratio
    clipped = -adv * torch.clamp(ratio, lower, upper)
    clip1 = torch.maximum(unclipped, clipped)
    dual = -adv * clip_c
    clip2 = torch.minimum(clip1, dual)
    tok = torch.where(adv < 0, clip2, clip1)
    klr = torch.zeros_like(tok)
    if kl_beta > 0.0 and ref_logp is not None:
        d = ref_logp - logp
        klr = torch.exp(d) - d - 1.0
        tok = tok + kl_beta * klr
    mf = mask.float()
    loss_sum = (tok * mf).sum()
    with torch.no_grad():
        lrd = lr.detach()
        rd = ratio.detach()
        z = torch.zeros_like(lrd)
        dual_active = (adv < 0) & (dual < clip1.detach())
        stats = torch.stack([
            mf.sum(), loss_sum.detach(), (lrd.abs() * mf).sum(), ((rd - 1 - lrd) * mf).sum(),
            ((rd > upper).float() * mf).sum(), ((rd < lower).float() * mf).sum(), (lrd * mf).sum(), (lrd * lrd * mf).sum(),
            ((entropy if entropy is not None else z) * mf).sum(), (adv * mf).sum(), (adv * adv * mf).sum(),
            ((adv > 0).float() * mf).sum(), ((adv == 0).float() * mf).sum(),
            ((clipped.detach() > unclipped.detach()).float() * mf).sum(),
            ((old_entropy if old_entropy is not None else z) * mf).sum(), (klr.detach() * mf).sum(),
            (logp.detach() * mf).sum(), (dual_active.float() * mf).sum(),
        ]).float()
    return loss_sum, stats


def adamw_step_(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor, lr: float, beta1: float,
                beta2: float, eps: float, wd: float, step: int, grad_scale: float = 1.0,
                max_norm: float = 0.0, norm_sq: Optional[torch.Tensor] = None) -> None:
    """In-place AdamW on fp32 tensors; clip coefficient min(1, max_norm / (sqrt(norm_sq) + 1e-6))."""
    coef = grad_scale
    if max_norm > 0.0 and norm_sq is not None:
        coef = coef * min(1.0, max_norm / (float(norm_sq.sqrt()) + 1e-6))
    gg = g * coef
    p.mul_(1.0 - lr * wd)
    m.mul_(beta1).add_(gg, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(gg, gg, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = v.sqrt() / math.sqrt(bc2) + eps
    p.addcdiv_(m, denom, value=-lr / bc1)


def normalize_rewards(rewards: Sequence[float]) -> List[float]:
    """Group-normalised advantages (r - mean) / (population std + 1e-4) (vllm_worker.py:788-796)."""
    n = len(rewards)
    if n == 0:
        return []
    mean = sum(rewards) / n
    var = sum((r - mean) ** 2 for r in rewards) / n
    std = math.sqrt(var)
    return [(r - mean) / (std + 1e-4) for r in rewards]


def stats_to_metrics(stats: Sequence[float], loss_value: float, num_samples: int, entropy_coeff: float = 0.0) -> Dict[str, float]:
    """Turn the sums vector into the reference's per-microbatch metric dict (grpo_loss.py:476-498)."""
    s = {k: float(v) for k, v in zip(LOSS_STAT_NAMES, stats)}
    n = max(1.0, s["count"])
    lr_mean = s["log_ratio"] / n
    lr_var = max(0.0, s["log_ratio_sq"] / n - lr_mean * lr_mean)
    adv_mean = s["adv"] / n
    adv_var = max(0.0, s["adv_sq"] / n - adv_mean * adv_mean)
    return {
        "loss": loss_value,
        "loss_per_token": loss_value / n if s["count"] > 0 else loss_value,
        "loss_per_sample": loss_value / num_samples if num_samples > 0 else loss_value,
        "pg_loss": loss_value,
        "pg_clip": s["pg_clip"],
        "kl_div": s["abs_log_ratio"] / n,
        "entropy": s["entropy"] / n,
        "old_policy_entropy": s["old_entropy"] / n,
        "entropy_coeff": float(entropy_coeff),
        "approx_kl": s["approx_kl"] / n,
        "clipfrac_upper": s["clip_upper"] / n,
        "clipfrac_lower": s["clip_lower"] / n,
        "log_ratio_mean": lr_mean,
        "log_ratio_std": math.sqrt(lr_var),
        "adv_mean": adv_mean,
        "adv_std": math.sqrt(adv_var),
        "adv_pos_frac": s["adv_pos"] / n,
        "adv_zero_frac": s["adv_zero"] / n,
        "kl_ref": s["kl_ref"] / n,
        "dual_clip_frac": s["dual_clip"] / n,
        "num_tokens": s["count"],
    }
