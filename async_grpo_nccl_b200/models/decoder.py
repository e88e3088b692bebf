"""Decoder forward / backward on the flat parameter layout.

Two executors over the SAME parameters and the SAME packed-batch contract:

* ``OracleDecoder``  - plain PyTorch (autograd), any device, any float dtype. It is the CPU plumbing
  path and the numerical oracle.
* ``NativeDecoder``  - sm_100a kernels with an explicit, hand-scheduled backward (no autograd graph):
  tcgen05 GEMMs with fused bias / residual epilogues, RMSNorm / RoPE / SwiGLU kernels, varlen
  flash-attention forward / backward, fused lm_head loss. Gradients accumulate in fp32 into a
  ``GradSink`` so the sharded optimizer can reduce them unit by unit.

Both replace the HF Qwen2 body + loss shim the reference runs (grpo_loss.py:40-144,
gpu_process_worker.py:963-1050).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, List, Optional, Tuple

import torch

from ..ops import reference as R
from ..packing import PackedBatch
from .config import ModelConfig
from .layout import ParamLayout


@dataclass
class LossConfig:
    clip_low: float = 0.2
    clip_high: float = 0.28
    clip_ratio_c: float = 3.0
    kl_beta: float = 0.0
    temperature: float = 1.0
    entropy_coeff: float = 0.0
    apply_entropy_bonus: bool = True


# =====================================================================================================
# Oracle
# =====================================================================================================
class OracleDecoder:
    def __init__(self, cfg: ModelConfig, layout: ParamLayout, params: torch.Tensor):
        self.cfg, self.layout, self.params = cfg, layout, params
        self._rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None

    def _rope_tables(self, device, need: int):
        if self._rope is None or self._rope[0].shape[0] < need or self._rope[0].device != device:
            n = max(need, min(self.cfg.max_position_embeddings, 4096))
            self._rope = R.rope_tables(self.cfg.head_dim, n, self.cfg.rope_theta, device)
        return self._rope

    def w(self, name: str) -> torch.Tensor:
        return self.layout.view(self.params, name)

    def hidden(self, ids: torch.Tensor, pos: torch.Tensor, cu_seqlens: List[int]) -> torch.Tensor:
        cfg = self.cfg
        cos_t, sin_t = self._rope_tables(ids.device, int(pos.max().item()) + 1 if pos.numel() else 1)
        x = self.w("embed")[ids.long()]
        T = x.shape[0]
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            h = R.rmsnorm(x, self.w(p + "ln1"), cfg.rms_norm_eps)
            qkv = h @ self.w(p + "wqkv").t()
            if cfg.attention_bias:
                qkv = qkv + self.w(p + "bqkv")
            q = qkv[:, :cfg.q_dim].reshape(T, cfg.num_attention_heads, cfg.head_dim)
            k = qkv[:, cfg.q_dim:cfg.q_dim + cfg.kv_dim].reshape(T, cfg.num_key_value_heads, cfg.head_dim)
            v = qkv[:, cfg.q_dim + cfg.kv_dim:].reshape(T, cfg.num_key_value_heads, cfg.head_dim)
            q = R.apply_rope(q, pos, cos_t, sin_t)
            k = R.apply_rope(k, pos, cos_t, sin_t)
            a = R.attention_varlen(q, k, v, cu_seqlens).reshape(T, cfg.q_dim)
            x = x + a @ self.w(p + "wo").t()
            h2 = R.rmsnorm(x, self.w(p + "ln2"), cfg.rms_norm_eps)
            x = x + R.swiglu(h2 @ self.w(p + "wgu").t()) @ self.w(p + "wd").t()
        return R.rmsnorm(x, self.w("final_norm"), cfg.rms_norm_eps)

    def logprobs(self, batch: PackedBatch, temperature: float) -> Tuple[torch.Tensor, torch.Tensor]:
        cu = batch.cu_seqlens.tolist()
        hn = self.hidden(batch.ids, batch.pos, cu)
        return R.lmhead_logprob_entropy(hn, self.w(self.layout.lm_head_name()), batch.labels, temperature)

    def loss(self, batch: PackedBatch, lc: LossConfig, loss_scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """Scaled microbatch loss (token mean * loss_scale) and the stats sums vector."""
        logp, ent = self.logprobs(batch, lc.temperature)
        ref = batch.ref_logprobs if lc.kl_beta > 0 else None
        loss_sum, stats = R.grpo_token_loss(logp, batch.old_logprobs, ref, batch.advantages, batch.labels, lc.clip_low,
                                            lc.clip_high, lc.clip_ratio_c, lc.kl_beta, ent, batch.old_entropies)
        denom = max(1.0, float(stats[0]))
        return loss_sum / denom * loss_scale, stats


# =====================================================================================================
# Native
# =====================================================================================================
class GradSink:
    """Where weight gradients go. ``unit_grads(u)`` returns an fp32 buffer covering unit ``u`` of the layout
    (kernels accumulate into it); ``unit_done(u)`` tells the owner that the unit's backward has finished."""

    def __init__(self, layout: ParamLayout, device, flat: Optional[torch.Tensor] = None):
        self.layout = layout
        self.flat = flat if flat is not None else torch.zeros(layout.total, dtype=torch.float32, device=device)

    def view(self, name: str) -> torch.Tensor:
        return self.layout.view(self.flat, name)

    def unit_done(self, unit: int) -> None:  # overridden by the sharded trainer
        pass

    def zero_(self) -> None:
        self.flat.zero_()


class NativeDecoder:
    def __init__(self, cfg: ModelConfig, layout: ParamLayout, params: Optional[torch.Tensor], recompute: bool = False,
                 lmhead_chunk: int = 4096, weights: Any = None):
        """``params`` is the resident flat bf16 parameter buffer. With ``weights`` (parallel/zero3.py::ShardedWeights)
        there is no resident copy: each unit is gathered from its owners just before use, the gather of the next unit
        riding on a GEMM launch of the current one."""
        from ..ops import native

        self.C = native()
        self.weights = weights
        if weights is None:
            assert params is not None and params.is_cuda and params.dtype == torch.bfloat16
            self.dev = params.device
        else:
            self.dev = weights.device
        self.cfg, self.layout, self.params = cfg, layout, params
        self.recompute = recompute
        self.lmhead_chunk = lmhead_chunk
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        if weights is not None:
            weights.status = self.status
        self._rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
        self.n_stats = int(self.C.grpo_num_loss_stats())
        self.launches = 0  # kernels of this package launched (bench bookkeeping)

    # ---- helpers ----
    def w(self, name: str) -> torch.Tensor:
        if self.weights is not None:
            return self.weights.view(name)
        return self.layout.view(self.params, name)

    def _enter_unit(self, unit: int, then: Optional[int]) -> None:
        """Sharded weights only: ``unit`` must be staged now; ``then`` is the unit needed after it (prefetched by the
        next large GEMM launch)."""
        if self.weights is not None:
            self.launches += self.weights.enter(unit, then)

    def rope_tables(self, need: int = 1):
        if self._rope is None or self._rope[0].shape[0] < need:
            n = max(need, min(self.cfg.max_position_embeddings, 131072))
            cos_t, sin_t = R.rope_tables(self.cfg.head_dim, n, self.cfg.rope_theta, "cpu")
            self._rope = (cos_t.to(self.dev), sin_t.to(self.dev))
        return self._rope

    def check_status(self) -> None:
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"device kernel reported status {code} (bounded wait ran out or bad index)")

    def _gemm(self, a, b, out, a_mn=False, b_mn=False, bias=None, accumulate=False, residual=None):
        if self.weights is not None and self.weights.wants_ride(a, b):
            self.weights.gemm_with_prefetch(a, b, out, a_mn, b_mn, bias, accumulate, self.status, residual)
        else:
            self.C.gemm_bf16(a, b, out, a_mn, b_mn, bias, 1.0, accumulate, self.status, residual)
        self.launches += 1
        return out

    def _wgrad(self, dy, x, name: str, sink) -> None:
        """dW[name] += dy^T x. A scatter sink adds the tile straight into the owners' gradient shards (GEMM fused with
        the reduce-scatter); the plain sink accumulates into the local fp32 buffer."""
        if getattr(sink, "scatter", False):
            sink.wgrad(dy, x, name, self.status)
        else:
            self.C.gemm_bf16(dy, x, sink.view(name), True, True, None, 1.0, True, self.status, None)
        self.launches += 1

    def _new(self, *shape, dtype=torch.bfloat16):
        return torch.empty(shape, dtype=dtype, device=self.dev)

    # ---- layer forward ----
    def _layer_fwd(self, i: int, x: torch.Tensor, batch: PackedBatch, cos_t, sin_t, save: Optional[dict],
                   kv_write: Optional[tuple] = None, next_unit: Optional[int] = None):
        cfg, C = self.cfg, self.C
        T = x.shape[0]
        p = f"layers.{i}."
        self._enter_unit(i + 1, next_unit)
        h1 = self._new(T, cfg.hidden_size)
        rstd1 = self._new(T, dtype=torch.float32)
        C.rmsnorm_fwd(x, self.w(p + "ln1"), h1, rstd1, cfg.rms_norm_eps)
        qkv = self._new(T, cfg.qkv_dim)
        self._gemm(h1, self.w(p + "wqkv"), qkv, bias=self.w(p + "bqkv") if cfg.attention_bias else None)
        C.rope_inplace(qkv, batch.pos, cos_t, sin_t, cfg.num_attention_heads + cfg.num_key_value_heads, cfg.head_dim, False)
        if kv_write is not None:  # rollout prefill: K/V of every prompt token go to their cache slots
            k_cache, v_cache, slots = kv_write[:3]
            head0 = kv_write[3] if len(kv_write) > 3 else 0  # tensor-parallel engine rank: its share of the kv heads
            C.kv_cache_write(qkv, slots, k_cache, v_cache, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                             self.status, head0)
            self.launches += 1
        attn = self._new(T, cfg.q_dim)
        lse = self._new(cfg.num_attention_heads, T, dtype=torch.float32)
        C.attn_varlen_fwd(qkv, attn, lse, batch.tiles, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                          1.0 / math.sqrt(cfg.head_dim), self.status)
        x1 = self._new(T, cfg.hidden_size)
        self._gemm(attn, self.w(p + "wo"), x1, residual=x)
        h2 = self._new(T, cfg.hidden_size)
        rstd2 = self._new(T, dtype=torch.float32)
        C.rmsnorm_fwd(x1, self.w(p + "ln2"), h2, rstd2, cfg.rms_norm_eps)
        gu = self._new(T, 2 * cfg.intermediate_size)
        self._gemm(h2, self.w(p + "wgu"), gu)
        act = self._new(T, cfg.intermediate_size)
        C.swiglu_fwd(gu, act)
        x2 = self._new(T, cfg.hidden_size)
        self._gemm(act, self.w(p + "wd"), x2, residual=x1)
        self.launches += 6
        if save is not None:
            save.update(x=x, h1=h1, rstd1=rstd1, qkv=qkv, attn=attn, lse=lse, x1=x1, h2=h2, rstd2=rstd2, gu=gu, act=act)
        return x2

    def layer_fwd_suffix(self, i: int, x: torch.Tensor, batch: PackedBatch, sfx: torch.Tensor, pfx: torch.Tensor,
                         pos_s: torch.Tensor, cos_t, sin_t, k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor,
                         pfx_blk: torch.Tensor, pfx_off: torch.Tensor) -> torch.Tensor:
        """Layer forward for a rollout prefill whose leading prompt tokens are already in the KV cache (prefix caching).
        ``x`` holds the rows of the tokens that still have to be computed (packed positions ``sfx`` of ``batch``, which
        describes the whole prompts). Projections and MLP run on those rows only; attention runs over the whole prompts
        with the keys / values of the cached tokens (packed positions ``pfx``, cache block / offset ``pfx_blk`` /
        ``pfx_off``) gathered from the cache. The query rows of cached tokens are zero and their outputs are dropped."""
        cfg, C = self.cfg, self.C
        Ts, T = x.shape[0], batch.T
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        p = f"layers.{i}."
        self._enter_unit(i + 1, None)
        h1 = self._new(Ts, cfg.hidden_size)
        C.rmsnorm_fwd(x, self.w(p + "ln1"), h1, None, cfg.rms_norm_eps)
        qkv_s = self._new(Ts, cfg.qkv_dim)
        self._gemm(h1, self.w(p + "wqkv"), qkv_s, bias=self.w(p + "bqkv") if cfg.attention_bias else None)
        C.rope_inplace(qkv_s, pos_s, cos_t, sin_t, Hq + Hkv, D, False)
        C.kv_cache_write(qkv_s, slots, k_cache, v_cache, Hq, Hkv, D, self.status, 0)
        qkv = torch.zeros(T, cfg.qkv_dim, dtype=torch.bfloat16, device=x.device)
        qkv.index_copy_(0, sfx, qkv_s)
        heads = qkv.view(T, Hq + 2 * Hkv, D)
        heads[pfx, Hq:Hq + Hkv] = k_cache[pfx_blk, :, pfx_off]   # [cached tokens, Hkv, D]
        heads[pfx, Hq + Hkv:] = v_cache[pfx_blk, :, pfx_off]
        attn = self._new(T, cfg.q_dim)
        lse = self._new(Hq, T, dtype=torch.float32)
        C.attn_varlen_fwd(qkv, attn, lse, batch.tiles, Hq, Hkv, D, 1.0 / math.sqrt(D), self.status)
        attn_s = attn.index_select(0, sfx)
        x1 = self._new(Ts, cfg.hidden_size)
        self._gemm(attn_s, self.w(p + "wo"), x1, residual=x)
        h2 = self._new(Ts, cfg.hidden_size)
        C.rmsnorm_fwd(x1, self.w(p + "ln2"), h2, None, cfg.rms_norm_eps)
        gu = self._new(Ts, 2 * cfg.intermediate_size)
        self._gemm(h2, self.w(p + "wgu"), gu)
        act = self._new(Ts, cfg.intermediate_size)
        C.swiglu_fwd(gu, act)
        x2 = self._new(Ts, cfg.hidden_size)
        self._gemm(act, self.w(p + "wd"), x2, residual=x1)
        self.launches += 12
        return x2

    def _layer_bwd(self, i: int, dx: torch.Tensor, s: dict, batch: PackedBatch, cos_t, sin_t, sink: GradSink):
        """dx (bf16 [T, H]) is the gradient w.r.t. the layer output; it is updated in place to the gradient w.r.t. the input."""
        cfg, C = self.cfg, self.C
        T = dx.shape[0]
        p = f"layers.{i}."
        self._enter_unit(i + 1, i if i > 0 else None)
        # ---- MLP ----
        dact = self._new(T, cfg.intermediate_size)
        self._gemm(dx, self.w(p + "wd"), dact, b_mn=True)
        self._wgrad(dx, s["act"], p + "wd", sink)
        dgu = self._new(T, 2 * cfg.intermediate_size)
        C.swiglu_bwd(s["gu"], dact, dgu)
        del dact
        dh2 = self._new(T, cfg.hidden_size)
        self._gemm(dgu, self.w(p + "wgu"), dh2, b_mn=True)
        self._wgrad(dgu, s["h2"], p + "wgu", sink)
        del dgu
        C.rmsnorm_bwd(dh2, s["x1"], self.w(p + "ln2"), s["rstd2"], dx, sink.view(p + "ln2"), True)
        # ---- attention ----
        dattn = self._new(T, cfg.q_dim)
        self._gemm(dx, self.w(p + "wo"), dattn, b_mn=True)
        self._wgrad(dx, s["attn"], p + "wo", sink)
        dqkv = self._new(T, cfg.qkv_dim)
        delta = self._new(cfg.num_attention_heads, T, dtype=torch.float32)
        dq_acc = self._new(T, cfg.q_dim, dtype=torch.float32)
        C.attn_varlen_bwd(s["qkv"], s["attn"], dattn, s["lse"], delta, dq_acc, dqkv, batch.tiles, cfg.num_attention_heads,
                          cfg.num_key_value_heads, cfg.head_dim, 1.0 / math.sqrt(cfg.head_dim), self.status)
        del dattn, delta, dq_acc
        C.rope_inplace(dqkv, batch.pos, cos_t, sin_t, cfg.num_attention_heads + cfg.num_key_value_heads, cfg.head_dim, True)
        if cfg.attention_bias:
            C.colsum(dqkv, sink.view(p + "bqkv"))
        dh1 = dh2  # reuse
        self._gemm(dqkv, self.w(p + "wqkv"), dh1, b_mn=True)
        self._wgrad(dqkv, s["h1"], p + "wqkv", sink)
        C.rmsnorm_bwd(dh1, s["x"], self.w(p + "ln1"), s["rstd1"], dx, sink.view(p + "ln1"), True)
        self.launches += 11
        sink.unit_done(i + 1)

    # ---- public ----
    def hidden(self, batch: PackedBatch, saves: Optional[List[dict]] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Returns (normed final hidden, pre-norm hidden, final rstd)."""
        cfg, C = self.cfg, self.C
        T = batch.T
        cos_t, sin_t = self.rope_tables()
        x = self._new(T, cfg.hidden_size)
        self._enter_unit(0, None)
        C.embedding_fwd(batch.ids, self.w("embed"), x)
        n_layers = cfg.num_hidden_layers
        for i in range(n_layers):
            save = None
            if saves is not None:
                save = {}
                saves.append(save)
            x_in = x
            x = self._layer_fwd(i, x, batch, cos_t, sin_t, save if not self.recompute else None,
                                next_unit=i + 2 if i + 1 < n_layers else None)
            if saves is not None and self.recompute:
                save["x"] = x_in
        hn = self._new(T, cfg.hidden_size)
        rstd = self._new(T, dtype=torch.float32)
        C.rmsnorm_fwd(x, self.w("final_norm"), hn, rstd, cfg.rms_norm_eps)
        self.launches += 2
        return hn, x, rstd

    def ensure_rope(self, max_pos: int) -> None:
        if self._rope is None or self._rope[0].shape[0] < max_pos:
            self._rope = None
            self.rope_tables(max_pos)

    def logprobs(self, batch: PackedBatch, temperature: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """Per-row logprob of the next token and entropy (fp32 [T]); forward only."""
        C = self.C
        hn, _, _ = self.hidden(batch)
        T = batch.T
        wl = self.w(self.layout.lm_head_name())
        groups = int(C.lmhead_num_groups(wl.shape[0], T))
        partials = self._new(3 * groups * T, dtype=torch.float32)
        ll = torch.zeros(T, dtype=torch.float32, device=self.dev)
        logp = self._new(T, dtype=torch.float32)
        ent = self._new(T, dtype=torch.float32)
        C.lmhead_logprob(hn, wl, batch.labels, temperature, partials, ll, logp, ent, None, self.status)
        self.launches += 2
        return logp, ent

    def forward_backward(self, batch: PackedBatch, lc: LossConfig, loss_scale: float, sink: GradSink) -> torch.Tensor:
        """One microbatch: forward, fused loss, full backward into ``sink``. Returns the device stats vector
        (sums over valid tokens, see ops.reference.LOSS_STAT_NAMES). The scalar loss is
        stats[loss_sum] / max(1, stats[count]) * loss_scale; nothing here synchronises with the host."""
        cfg, C = self.cfg, self.C
        T = batch.T
        cos_t, sin_t = self.rope_tables()
        saves: List[dict] = []
        hn, x_last, rstd_f = self.hidden(batch, saves)
        wl_name = self.layout.lm_head_name()
        wl = self.w(wl_name)
        V = wl.shape[0]
        groups = int(C.lmhead_num_groups(V, T))
        partials = self._new(3 * groups * T, dtype=torch.float32)
        ll = torch.zeros(T, dtype=torch.float32, device=self.dev)
        logp = self._new(T, dtype=torch.float32)
        ent = self._new(T, dtype=torch.float32)
        lse = self._new(T, dtype=torch.float32)
        C.lmhead_logprob(hn, wl, batch.labels, lc.temperature, partials, ll, logp, ent, lse, self.status)
        del partials
        stats = torch.zeros(self.n_stats, dtype=torch.float32, device=self.dev)
        dlogp = self._new(T, dtype=torch.float32)
        n_valid = max(1.0, batch.scalars.get("num_output_tokens_non_masked", float(batch.total_out)))
        ref = batch.ref_logprobs if (lc.kl_beta > 0 and batch.has_ref) else None
        C.grpo_token_loss(logp, batch.old_logprobs, ref, batch.advantages, batch.labels, ent, batch.old_entropies,
                          lc.clip_low, lc.clip_high, lc.clip_ratio_c, lc.kl_beta, loss_scale / n_valid, dlogp, stats)
        chunk = min(self.lmhead_chunk, (V + 255) // 256 * 256)
        dz = self._new(T, chunk)
        dh_acc = self._new(T, cfg.hidden_size, dtype=torch.float32)
        C.lmhead_backward(hn, wl, batch.labels, lse, dlogp, lc.temperature, dz, dh_acc, sink.view(wl_name), self.status)
        del dz
        dhn = self._new(T, cfg.hidden_size)
        C.cast_f32_bf16(dh_acc, dhn)
        del dh_acc
        dx = self._new(T, cfg.hidden_size)
        C.rmsnorm_bwd(dhn, x_last, self.w("final_norm"), rstd_f, dx, sink.view("final_norm"), False)
        del dhn
        self.launches += 8 + 3 * ((V + chunk - 1) // chunk)
        for i in reversed(range(cfg.num_hidden_layers)):
            s = saves[i]
            if self.recompute:
                full: dict = {}
                self._layer_fwd(i, s["x"], batch, cos_t, sin_t, full, next_unit=i if i > 0 else None)
                s = full
            self._layer_bwd(i, dx, s, batch, cos_t, sin_t, sink)
            saves[i] = None  # free activations of this layer
        C.embedding_bwd(batch.ids, dx, sink.view("embed"))
        self.launches += 1
        sink.unit_done(0)
        return stats
