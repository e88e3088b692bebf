"""Native rollout engine: continuous batching over a paged KV cache.

It provides what the reference gets from vLLM's ``AsyncLLM`` (vllm_worker.py:203-284, 709-737): one
request per prompt with ``n`` samples, temperature sampling with a per-request seed, a cap on new
tokens, EOS stopping, and prompt-prefix sharing between the ``n`` samples of a group (the prompt is
prefetched once; only its partial last block is copied per sample).

* scheduling / block accounting: C++ (``csrc/host/kv_allocator.cpp``)
* prefill: packed varlen forward through the same decoder kernels as training, K/V written to the pages
* decode: one fused step per token for all running sequences (skinny tcgen05 GEMMs, paged-KV GQA
  attention, lm_head + Gumbel-max sampling without materialising logits), optionally replayed from a
  CUDA graph (preset ``throughput``)

``OracleEngine`` offers the same API on any device with plain PyTorch (used by the CPU plumbing
configuration and as the greedy-decoding oracle in tests).
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.config import ModelConfig
from ..models.decoder import NativeDecoder, OracleDecoder
from ..models.layout import ParamLayout
from ..packing import pack_samples

GOLDEN = 0x9E3779B97F4A7C15


@dataclass
class FinishedSequence:
    request_id: Any
    child: int
    output_ids: np.ndarray  # int32
    finish_reason: str  # "stop" (EOS) | "length"
    prompt_len: int
    output_logprobs: Optional[np.ndarray] = None  # fp32 log-probability of every sampled token (when recorded)


@dataclass
class _Request:
    request_id: Any
    prompt: np.ndarray
    n: int
    max_new_tokens: int
    temperature: float
    seed: int
    forced_new_tokens: Optional[List[int]]
    ignore_eos: bool
    group_id: int = -1
    child_map: Optional[List[int]] = None  # original child indices when a request is a re-queued remainder


def _mix_seed(seed: int, child: int) -> int:
    x = (seed * 0x2545F4914F6CDD1D + (child + 1) * GOLDEN) & 0xFFFFFFFFFFFFFFFF
    x ^= x >> 29
    return x & 0x7FFFFFFFFFFFFFFF


class RolloutEngine:
    def __init__(self, cfg: ModelConfig, layout: ParamLayout, params: torch.Tensor, *, max_seqs: int = 256,
                 max_model_len: Optional[int] = None, num_blocks: Optional[int] = None, block_size: int = 16,
                 kv_memory_bytes: Optional[int] = None, max_prefill_tokens: int = 16384, use_cuda_graph: bool = False,
                 eos_token_id: Optional[int] = None, tp: Any = None, prefix_caching: bool = False):
        from ..ops import native

        assert params.is_cuda and params.dtype == torch.bfloat16
        if block_size != 16 or cfg.head_dim != 128:
            raise ValueError("the native engine supports block_size 16 and head_dim 128")
        self.C = native()
        self.cfg, self.layout, self.params = cfg, layout, params
        self.dev = params.device
        # Tensor parallelism (vllm_worker.py:219-232, tensor_parallel_size): ``tp`` is a parallel.symm.TensorParallelComm.
        # This rank then holds Hq / tp query heads and Hkv / tp kv heads (projection columns, KV cache) and F / tp MLP
        # columns; the o and down projections produce partial sums that are all-reduced over peer memory. Embedding,
        # lm_head and sampling are replicated: every member computes the same token from the same bits.
        self.tp = tp if (tp is not None and tp.size > 1) else None
        self.tp_size = self.tp.size if self.tp is not None else 1
        self.tp_rank = self.tp.rank if self.tp is not None else 0
        t = self.tp_size
        if cfg.num_attention_heads % t or cfg.num_key_value_heads % t or cfg.intermediate_size % (8 * t):
            raise ValueError(f"tensor parallel size {t} must divide the head counts and the MLP width")
        self.Hq_l, self.Hkv_l, self.F_l = cfg.num_attention_heads // t, cfg.num_key_value_heads // t, cfg.intermediate_size // t
        self.Q_l = (self.Hq_l + 2 * self.Hkv_l) * cfg.head_dim
        self.qd_l = self.Hq_l * cfg.head_dim
        # Prefix caching across requests (vllm_worker.py:224, enable_prefix_caching): full prompt blocks stay findable by
        # the hash of their token chain after their last user has gone; a later prompt that starts with the same chain
        # reuses them and only its remaining tokens go through the GEMMs. Forgotten at every weight update. A
        # tensor-parallel member caches only its own kv heads while the prefill needs all of them, so it stays off there.
        self.prefix_caching = bool(prefix_caching) and self.tp is None
        self.prefix_hit_tokens = 0
        self.prefix_lookup_tokens = 0
        self.sm_count = torch.cuda.get_device_properties(self.dev).multi_processor_count  # SMs the engine's stream may use
        self.dec = NativeDecoder(cfg, layout, params)
        self.status = self.dec.status
        self.block_size = block_size
        self.max_seqs = int(max_seqs)
        self.max_model_len = int(max_model_len or cfg.max_position_embeddings)
        self.max_blocks_per_seq = (self.max_model_len + block_size - 1) // block_size
        self.eos = cfg.eos_token_id if eos_token_id is None else int(eos_token_id)
        per_block = cfg.num_hidden_layers * 2 * self.Hkv_l * block_size * cfg.head_dim * 2
        if num_blocks is None:
            if kv_memory_bytes is None:
                free, _ = torch.cuda.mem_get_info(self.dev)
                kv_memory_bytes = int(free * 0.6)
            num_blocks = max(64, kv_memory_bytes // per_block)
        self.num_blocks = int(num_blocks)
        self.cache = torch.zeros(cfg.num_hidden_layers, 2, self.num_blocks, self.Hkv_l, block_size,
                                 cfg.head_dim, dtype=torch.bfloat16, device=self.dev)
        self.sched = self.C.Scheduler(self.num_blocks, block_size, self.max_seqs, self.max_blocks_per_seq,
                                      int(max_prefill_tokens))
        self.dec.ensure_rope(min(self.max_model_len, cfg.max_position_embeddings))
        S, H = self.max_seqs, cfg.hidden_size
        i32 = dict(dtype=torch.int32, device=self.dev)
        bf = dict(dtype=torch.bfloat16, device=self.dev)
        self.block_tables = torch.zeros(S, self.max_blocks_per_seq, **i32)
        self.seq_lens = torch.zeros(S, **i32)
        self.positions = torch.zeros(S, **i32)
        self.last_tokens = torch.zeros(S, **i32)
        self.gen_index = torch.zeros(S, dtype=torch.int64, device=self.dev)
        self.base_seeds = torch.zeros(S, dtype=torch.int64, device=self.dev)
        self.step_seeds = torch.zeros(S, dtype=torch.int64, device=self.dev)
        self.row_ids = torch.arange(S, dtype=torch.int64, device=self.dev)
        self.hist_cap = self.max_model_len
        self.history = torch.zeros(S, self.hist_cap, **i32)
        # decode activations (persistent: no allocation inside a step, required for graph capture); the persistent
        # layer kernel loads them in row tiles of 32 / 64 / 128 / 256, so the buffers hold at least the tile that covers S
        SA = next((t for t in (32, 64, 128, 256) if t >= S), S)
        self.b_x = torch.zeros(SA, H, **bf)
        self.b_x1 = torch.zeros(SA, H, **bf)
        self.b_h = torch.empty(S, H, **bf)
        self.b_qkv = torch.zeros(SA, self.Q_l, **bf)
        self.b_attn = torch.zeros(SA, self.qd_l, **bf)
        self.b_gu = torch.empty(S, 2 * self.F_l, **bf)
        self.b_act = torch.zeros(SA, self.F_l, **bf)
        self.b_tokens = torch.zeros(S, **i32)
        self.max_splits = 8
        self.b_part_o = torch.empty(S * cfg.num_key_value_heads * self.max_splits * 8 * cfg.head_dim, dtype=torch.float32,
                                    device=self.dev)
        self.b_part_ml = torch.empty(S * cfg.num_key_value_heads * self.max_splits * 16, dtype=torch.float32, device=self.dev)
        # arrival counters of the split-KV merge (the last split CTA merges; counters re-arm themselves)
        self.b_tickets = torch.zeros(S * cfg.num_key_value_heads, dtype=torch.int32, device=self.dev)
        groups = int(self.C.lm_sample_num_groups(cfg.vocab_size, S))
        g_small = max(groups, int(self.C.lm_sample_num_groups(cfg.vocab_size, 1)))
        self.b_sample_f = torch.empty(4 * g_small * S, dtype=torch.float32, device=self.dev)
        self.b_sample_i = torch.empty(g_small * S, **i32)
        # host mirrors (one entry per slot); all per-step bookkeeping on them is vectorised
        self.h_lens = np.zeros(S, np.int32)
        self.h_gen = np.zeros(S, np.int64)
        self.h_seq = np.full(S, -1, np.int64)            # sequence id living in the slot, -1 = free
        self.h_limit = np.full(S, 1 << 60, np.int64)     # number of generated tokens at which the sequence ends
        self.h_watch = np.zeros(S, bool)                  # stop at EOS?
        self.h_eos_at = np.full(S, -1, np.int64)         # index of the generated EOS token, -1 = none seen
        self.n_watch = 0
        # every decode step's inputs (lengths, block-table updates, seed increment) travel in one pinned staging buffer;
        # the host runs ahead of the device, so there is a ring of them, each reused only after its copy completed
        self.stage_ring = [torch.zeros(3 * S + 4, dtype=torch.int32).pin_memory() for _ in range(8)]
        self.stage_np = [t.numpy() for t in self.stage_ring]
        self.stage_events = [torch.cuda.Event() for _ in range(8)]
        self.d_stage = torch.zeros(3 * S + 4, dtype=torch.int32, device=self.dev)
        self.h_tok_pin = [torch.zeros(S, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.tok_events = [torch.cuda.Event(), torch.cuda.Event()]
        self.tok_pending: List[Optional[List[Tuple[int, int, int]]]] = [None, None]
        self.step_count = 0
        self.launches = 0
        # host-side time accounting of the step loop (seconds): where a step's wall time goes on the CPU
        self.t_plan = self.t_prep = self.t_launch = self.t_post = self.t_prefill = self.t_wait = 0.0
        self.n_decode_steps = self.n_prefill_steps = 0
        # ---- fused decode path (batches of up to 256 rows) ----
        # RMSNorm weights are folded into the columns of the matrices that consume the normalised rows (private copies
        # of wqkv and wgu, refreshed after every weight sync); the row scale rsqrt(mean(x^2) + eps) is applied in those
        # GEMMs' epilogues from sums of squares that the producing GEMMs' epilogues accumulate. Together with the fused
        # gate/up + SwiGLU GEMM a layer is 6 kernels instead of 9.
        L, F, Q = cfg.num_hidden_layers, self.F_l, self.Q_l   # this rank's share under tensor parallelism
        self.fused_chunk = min(256, self.max_seqs)   # rows per launch of the skinny GEMMs
        self.fused_decode = F % 8 == 0 and all(
            int(self.C.gemm_skinny_splits(m, n, k)) > 0
            for m in range(32, self.fused_chunk + 1, 32) for n, k in ((Q, H), (H, self.qd_l), (H, F)))
        if self.tp is not None:
            if not self.fused_decode or self.max_seqs > self.fused_chunk:
                raise ValueError("the tensor-parallel engine needs the fused decode path and at most 256 sequences per replica")
            self.bq_local = torch.zeros(L, Q, **bf)
        self.fused_rows = self.max_seqs if self.fused_decode else 0  # larger batches go through in chunks
        if self.fused_decode:
            self.folded = torch.empty(L * (Q + 2 * F) * H, **bf)
            self.b_ss = torch.zeros(2 * L + 1, S, dtype=torch.int64, device=self.dev)  # fixed point, value * 2^30
            self.refold_weights()
        # ---- persistent layer kernel: every decoder layer of a step in one cooperative launch (up to 256 rows) ----
        self.mega_rows = 0
        self.mega_trace: Optional[torch.Tensor] = None  # int64[32]: phase stamps of CTA 0 in layer mega_trace_layer
        self.mega_trace_layer = 0
        if (self.fused_decode and self.tp is None and os.environ.get("AGRPO_DECODE_MEGA", "1") != "0"
                and self.C.decode_layers_supported(min(256, S), H, Q, cfg.q_dim, F, cfg.num_attention_heads,
                                                   cfg.num_key_value_heads, cfg.head_dim)):
            # it wins where the step is latency-bound (few rows); with more rows both paths are bound by streaming the
            # KV cache and the per-phase hand-offs of the persistent kernel cost more than separate launches
            self.mega_rows = min(int(os.environ.get("AGRPO_MEGA_MAX_ROWS", "32")), 256, S)
            seg = self.layout.segments
            nxt = 1 if L > 1 else 0
            self.mega_strides = {k: seg[f"layers.{nxt}.{k}"].offset - seg[f"layers.0.{k}"].offset
                                 for k in (("wo", "wd", "bqkv") if cfg.attention_bias else ("wo", "wd"))}
            uniform = all(seg[f"layers.{i}.{k}"].offset - seg[f"layers.0.{k}"].offset == i * st
                          for k, st in self.mega_strides.items() for i in range(L))
            if not uniform:
                self.mega_rows = 0
            else:
                self.b_partials = torch.empty(int(self.C.decode_layers_scratch_bytes(self.mega_rows, H, Q, cfg.q_dim, F)) // 4,
                                              dtype=torch.float32, device=self.dev)
                self.b_counters = torch.zeros(int(self.C.decode_layers_counter_words()), **i32)
        # chosen-token log-probabilities (off until a caller asks: one more small tensor op per step)
        self.record_logprobs = False
        self.b_lp: Optional[torch.Tensor] = None
        self.history_lp: Optional[torch.Tensor] = None
        self.use_cuda_graph = use_cuda_graph
        self.use_pdl = os.environ.get("AGRPO_DECODE_PDL", "1") != "0"
        # keep running sequences in a dense prefix of the slots: the decode batch has as many rows as the highest slot
        self.compact_slots = os.environ.get("AGRPO_COMPACT_SLOTS", "1") != "0"
        self.n_compactions = 0
        self._last_rows = self._last_active = 0
        self.graphs: Dict[Tuple[int, float, int], torch.cuda.CUDAGraph] = {}
        self.requests: Dict[int, _Request] = {}
        self.slot_info: Dict[int, Dict[str, Any]] = {}
        self.pending: List[_Request] = []
        self.next_group = 0
        self.temperature: Optional[float] = None
        self.tokens_generated = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ------------------------------------------------------------------ requests
    def add_request(self, request_id: Any, prompt_ids: Sequence[int], n: int = 1, max_new_tokens: int = 128,
                    temperature: float = 1.0, seed: int = 0, forced_new_tokens: Optional[Sequence[int]] = None,
                    ignore_eos: bool = False) -> None:
        prompt = np.ascontiguousarray(np.asarray(prompt_ids, dtype=np.int32))
        room = self.max_model_len - len(prompt) - 1
        max_new = max(1, min(int(max_new_tokens), room))
        forced = None
        if forced_new_tokens is not None:
            forced = [max(1, min(int(f), max_new)) for f in forced_new_tokens]
        self.pending.append(_Request(request_id, prompt, int(n), max_new, float(temperature), int(seed), forced,
                                     bool(ignore_eos or forced is not None)))

    def enable_logprobs(self) -> None:
        """From now on the log-probability of every sampled token (under the sampling temperature) is kept next to the
        token history and returned with finished sequences (what the reference reads from vLLM's ``logprobs`` output,
        vllm_worker.py:286-392). Captured graphs are dropped: the step gains one output."""
        if self.record_logprobs:
            return
        self.record_logprobs = True
        self.b_lp = torch.zeros(self.max_seqs, dtype=torch.float32, device=self.dev)
        self.history_lp = torch.zeros(self.max_seqs, self.hist_cap, dtype=torch.float32, device=self.dev)
        self.graphs.clear()

    def has_work(self) -> bool:
        return bool(self.pending) or self.sched.num_waiting > 0 or self.sched.num_running > 0

    def _admit_pending(self) -> None:
        keep = []
        for r in self.pending:
            if self.temperature is None or self.sched.num_running == 0 and self.sched.num_waiting == 0:
                self.temperature = r.temperature
            if r.temperature != self.temperature:
                keep.append(r)
                continue
            r.group_id = self.next_group
            self.next_group += 1
            self.requests[r.group_id] = r
            self.sched.add_group(r.group_id, len(r.prompt), r.n, r.max_new_tokens, r.forced_new_tokens or [],
                                 self._block_hashes(r.prompt) if self.prefix_caching else [])
        self.pending = keep

    def _block_hashes(self, prompt: np.ndarray) -> List[int]:
        """Hash of the token chain up to and including every full block of the prompt (64 bits, never 0)."""
        import hashlib

        out: List[int] = []
        prev = b"agrpo-prefix"
        bs = self.block_size
        for b in range(len(prompt) // bs):
            prev = hashlib.blake2b(prev + prompt[b * bs:(b + 1) * bs].tobytes(), digest_size=8).digest()
            out.append(int.from_bytes(prev, "little") or 1)
        return out

    # ------------------------------------------------------------------ model pieces
    def _kc(self, i: int) -> torch.Tensor:
        return self.cache[i, 0]

    def _vc(self, i: int) -> torch.Tensor:
        return self.cache[i, 1]

    def _apply_table_updates(self, plan: Dict[str, Any]) -> None:
        n = len(plan["upd_slot"])
        if n == 0:
            return
        u = torch.tensor([plan["upd_slot"], plan["upd_index"], plan["upd_block"]], dtype=torch.int64).pin_memory()
        ud = u.to(self.dev, non_blocking=True)
        self.h2d_bytes += u.numel() * 8
        self.block_tables.index_put_((ud[0], ud[1]), ud[2].to(torch.int32))

    def _sample(self, hidden: torch.Tensor, rows: int, seeds: torch.Tensor, tokens: torch.Tensor, temperature: float,
                logprobs: Optional[torch.Tensor] = None) -> None:
        wl = self.layout.view(self.params, self.layout.lm_head_name())
        self.C.lm_sample(hidden[:rows], wl, temperature, seeds, self.b_sample_f, self.b_sample_i, tokens, logprobs, self.status)
        self.launches += 2

    def _prefill(self, plan: Dict[str, Any]) -> None:
        cfg, C, dec = self.cfg, self.C, self.dec
        gids = plan["group_ids"]
        reqs = [self.requests[g] for g in gids]
        samples = [{"sample_ids": r.prompt, "input_len": len(r.prompt), "output_len": 0, "advantage": 0.0} for r in reqs]
        host_batch = pack_samples(samples, pin=True)
        batch = host_batch.to_device(self.dev)
        slots = torch.tensor(plan["slot_mapping"], dtype=torch.int32).pin_memory().to(self.dev, non_blocking=True)
        self.h2d_bytes += host_batch.h2d_bytes() + slots.numel() * 4 + 16 * len(plan["seq_slots"])
        self._apply_table_updates(plan)
        cos_t, sin_t = dec.rope_tables(1)
        T = batch.T
        cached = plan.get("cached_lens") or []
        if self.prefix_caching:
            self.prefix_lookup_tokens += T
            self.prefix_hit_tokens += int(sum(cached))
        if any(cached):
            xl = self._prefill_suffix(plan, batch, slots, cached, cos_t, sin_t)
        else:
            x = torch.empty(T, cfg.hidden_size, dtype=torch.bfloat16, device=self.dev)
            C.embedding_fwd(batch.ids, dec.w("embed"), x)
            for i in range(cfg.num_hidden_layers):
                x = dec._layer_fwd(i, x, batch, cos_t, sin_t, None, kv_write=(self._kc(i), self._vc(i), slots, self.tp_rank * self.Hkv_l))
            last = (batch.cu_seqlens[1:] - 1).long()
            xl = x.index_select(0, last)
        hn = torch.empty_like(xl)
        C.rmsnorm_fwd(xl, dec.w("final_norm"), hn, None, cfg.rms_norm_eps)
        if plan["copy_src"]:
            src = torch.tensor(plan["copy_src"], dtype=torch.int64).pin_memory().to(self.dev, non_blocking=True)
            dst = torch.tensor(plan["copy_dst"], dtype=torch.int64).pin_memory().to(self.dev, non_blocking=True)
            self.cache[:, :, dst] = self.cache[:, :, src]
        # one sampling row per child
        rep = torch.tensor([r.n for r in reqs], dtype=torch.int64, device=self.dev)
        hrep = hn.repeat_interleave(rep, dim=0).contiguous()
        seq_slots = plan["seq_slots"]
        n_rows = len(seq_slots)
        seeds_host = []
        k = 0
        for r in reqs:
            for c in range(r.n):
                seeds_host.append(_mix_seed(r.seed, r.child_map[c] if r.child_map else c))
                slot = seq_slots[k]
                forced = r.forced_new_tokens[c] if r.forced_new_tokens else None
                child = r.child_map[c] if r.child_map else c
                self.slot_info[slot] = {"seq_id": plan["seq_ids"][k], "req": r, "child": child, "forced": forced}
                self.h_lens[slot] = len(r.prompt)
                self.h_gen[slot] = 1
                self.h_seq[slot] = plan["seq_ids"][k]
                self.h_limit[slot] = forced if forced is not None else r.max_new_tokens
                self.h_watch[slot] = not r.ignore_eos
                self.h_eos_at[slot] = -1
                self.n_watch += int(not r.ignore_eos)
                k += 1
        seeds = torch.tensor(seeds_host, dtype=torch.int64).pin_memory().to(self.dev, non_blocking=True)
        slot_idx = torch.tensor(seq_slots, dtype=torch.int64).pin_memory().to(self.dev, non_blocking=True)
        toks = torch.empty(n_rows, dtype=torch.int32, device=self.dev)
        lps = torch.empty(n_rows, dtype=torch.float32, device=self.dev) if self.record_logprobs else None
        # rows are processed in pieces of at most max_seqs so the scratch buffers suffice
        for s in range(0, n_rows, self.max_seqs):
            e = min(n_rows, s + self.max_seqs)
            self._sample(hrep[s:e], e - s, seeds[s:e], toks[s:e], self.temperature or 0.0, lps[s:e] if lps is not None else None)
        self.base_seeds.index_copy_(0, slot_idx, seeds)
        self.last_tokens.index_copy_(0, slot_idx, toks)
        self.history[slot_idx, 0] = toks
        if lps is not None:
            self.history_lp[slot_idx, 0] = lps
        self.gen_index.index_fill_(0, slot_idx, 1)
        self.tokens_generated += n_rows
        self.launches += dec.launches
        dec.launches = 0
        if not all(r.ignore_eos for r in reqs):
            th = toks.cpu().numpy()
            for j, slot in enumerate(seq_slots):
                if self.h_watch[slot] and int(th[j]) == self.eos:
                    self.h_eos_at[slot] = 0

    def _prefill_suffix(self, plan: Dict[str, Any], batch: Any, slots: torch.Tensor, cached: Sequence[int], cos_t, sin_t) -> torch.Tensor:
        """Prefill of prompts whose leading blocks came from the prefix cache: only the remaining tokens go through the
        projections and the MLP; their attention runs over the whole prompt, with the keys and values of the cached
        tokens gathered from the cache. Returns the hidden state of every prompt's last token."""
        cfg, C, dec = self.cfg, self.C, self.dec
        cu = np.concatenate([[0], np.cumsum(np.asarray(plan["prompt_lens"], dtype=np.int64))])  # prompts are packed in order
        sfx_parts, pfx_parts, last_s = [], [], []
        n_s = 0
        for g, c in enumerate(cached):
            a, b = int(cu[g]), int(cu[g + 1])
            pfx_parts.append(np.arange(a, a + int(c), dtype=np.int64))
            sfx_parts.append(np.arange(a + int(c), b, dtype=np.int64))
            n_s += b - a - int(c)
            last_s.append(n_s - 1)
        idx_host = torch.from_numpy(np.concatenate(sfx_parts + pfx_parts + [np.asarray(last_s, dtype=np.int64),
                                                                           np.asarray(plan["prefix_slots"], dtype=np.int64)]))
        idx = idx_host.pin_memory().to(self.dev, non_blocking=True)
        self.h2d_bytes += idx.numel() * 8
        n_p = int(sum(int(c) for c in cached))
        sfx, pfx = idx[:n_s], idx[n_s:n_s + n_p]
        last = idx[n_s + n_p:n_s + n_p + len(cached)]
        pslots = idx[n_s + n_p + len(cached):]
        ids_s = batch.ids.index_select(0, sfx)
        pos_s = batch.pos.index_select(0, sfx)
        x = torch.empty(n_s, cfg.hidden_size, dtype=torch.bfloat16, device=self.dev)
        C.embedding_fwd(ids_s, dec.w("embed"), x)
        blk, off = pslots // self.block_size, pslots % self.block_size
        for i in range(cfg.num_hidden_layers):
            x = dec.layer_fwd_suffix(i, x, batch, sfx, pfx, pos_s, cos_t, sin_t, self._kc(i), self._vc(i), slots, blk, off)
        return x.index_select(0, last)

    def _decode_forward(self, B: int, temperature: float, splits: int) -> None:
        if self.mega_rows and B <= self.mega_rows:
            return self._decode_forward_mega(B, temperature, splits)
        if self.fused_decode and B <= self.fused_rows:
            # short kernels back to back: let each prologue overlap the tail of the kernel before (this thread only)
            self.C.set_pdl(self.use_pdl)
            try:
                return self._decode_forward_fused(B, temperature, splits)
            finally:
                self.C.set_pdl(False)
        cfg, C, dec = self.cfg, self.C, self.dec
        cos_t, sin_t = dec.rope_tables(1)
        x, x1, h, qkv, attn, gu, act = (self.b_x[:B], self.b_x1[:B], self.b_h[:B], self.b_qkv[:B], self.b_attn[:B],
                                        self.b_gu[:B], self.b_act[:B])
        bt, sl = self.block_tables, self.seq_lens
        scale = 1.0 / math.sqrt(cfg.head_dim)
        C.embedding_fwd(self.last_tokens[:B], dec.w("embed"), x)
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            C.rmsnorm_fwd(x, dec.w(p + "ln1"), h, None, cfg.rms_norm_eps)
            C.gemm_bf16(h, dec.w(p + "wqkv"), qkv, False, False, dec.w(p + "bqkv") if cfg.attention_bias else None, 1.0, False,
                        self.status, None)
            C.rope_kv_write_decode(qkv, cos_t, sin_t, bt, sl, self._kc(i), self._vc(i), cfg.num_attention_heads,
                                   cfg.num_key_value_heads, cfg.head_dim, self.status)
            C.paged_decode_attn(qkv, self._kc(i), self._vc(i), bt, sl, attn, cfg.num_attention_heads, cfg.num_key_value_heads,
                                cfg.head_dim, scale, splits, self.b_part_o, self.b_part_ml, self.status, self.b_tickets)
            C.gemm_bf16(attn, dec.w(p + "wo"), x1, False, False, None, 1.0, False, self.status, x)
            C.rmsnorm_fwd(x1, dec.w(p + "ln2"), h, None, cfg.rms_norm_eps)
            C.gemm_bf16(h, dec.w(p + "wgu"), gu, False, False, None, 1.0, False, self.status, None)
            C.swiglu_fwd(gu, act)
            C.gemm_bf16(act, dec.w(p + "wd"), x, False, False, None, 1.0, False, self.status, x1)
        C.rmsnorm_fwd(x, dec.w("final_norm"), h, None, cfg.rms_norm_eps)
        wl = self.layout.view(self.params, self.layout.lm_head_name())
        C.lm_sample(h, wl, temperature, self.step_seeds, self.b_sample_f, self.b_sample_i, self.b_tokens, self.b_lp, self.status)
        self._feed_back(B)

    def _feed_back(self, B: int) -> None:
        """The sampled token becomes the next step's input and goes into the history (with its log-probability when kept)."""
        pos = torch.clamp(self.gen_index[:B], max=self.hist_cap - 1)
        self.last_tokens[:B].copy_(self.b_tokens[:B])
        self.history[self.row_ids[:B], pos] = self.b_tokens[:B]
        if self.record_logprobs:
            self.history_lp[self.row_ids[:B], pos] = self.b_lp[:B]
        self.gen_index[:B].add_(1)

    # ---- fused decode path ----
    def _folded(self, i: int) -> Tuple[torch.Tensor, torch.Tensor]:
        cfg = self.cfg
        H, F, Q = cfg.hidden_size, self.F_l, self.Q_l
        per = (Q + 2 * F) * H
        base = i * per
        return (self.folded[base: base + Q * H].view(Q, H), self.folded[base + Q * H: base + per].view(2 * F, H))

    def refold_weights(self) -> None:
        """Recomputes the norm-folded copies of wqkv and wgu from the current parameters (2 small kernels per layer)."""
        if not self.fused_decode:
            return
        dec, C, cfg = self.dec, self.C, self.cfg
        if self.tp is not None:
            return self._refold_weights_tp()
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            fq, fg = self._folded(i)
            C.fold_norm_weight(dec.w(p + "wqkv"), dec.w(p + "ln1"), fq)
            C.fold_norm_weight(dec.w(p + "wgu"), dec.w(p + "ln2"), fg)
        self.launches += 2 * cfg.num_hidden_layers

    def _refold_weights_tp(self) -> None:
        """This rank's rows of wqkv (its q, k and v heads) and of wgu (its gate and up columns), norm-folded, plus its
        slice of the qkv bias."""
        dec, C, cfg = self.dec, self.C, self.cfg
        r, D = self.tp_rank, cfg.head_dim
        qd, kvd, F = cfg.q_dim, cfg.kv_dim, cfg.intermediate_size
        ql, kl, fl = self.qd_l, self.Hkv_l * D, self.F_l
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            fq, fg = self._folded(i)
            wq, wg = dec.w(p + "wqkv"), dec.w(p + "wgu")
            ln1, ln2 = dec.w(p + "ln1"), dec.w(p + "ln2")
            rows = ((r * ql, ql), (qd + r * kl, kl), (qd + kvd + r * kl, kl))
            o = 0
            for a, n in rows:
                C.fold_norm_weight(wq[a:a + n], ln1, fq[o:o + n])
                if cfg.attention_bias:
                    self.bq_local[i, o:o + n].copy_(dec.w(p + "bqkv")[a:a + n])
                o += n
            C.fold_norm_weight(wg[r * fl:(r + 1) * fl], ln2, fg[:fl])
            C.fold_norm_weight(wg[F + r * fl:F + (r + 1) * fl], ln2, fg[fl:])
        self.launches += 5 * cfg.num_hidden_layers

    def _decode_forward_fused(self, B: int, temperature: float, splits: int) -> None:
        """Five kernels per layer for up to 256 rows. Larger batches run layer by layer in row chunks of at most 256: a
        layer's weights (tens of MB) are still in L2 when the second chunk reads them, so they cross HBM once."""
        cfg, C, dec = self.cfg, self.C, self.dec
        cos_t, sin_t = dec.rope_tables(1)
        ss = self.b_ss
        scale = 1.0 / math.sqrt(cfg.head_dim)
        eps = cfg.rms_norm_eps
        st = self.status
        R = self.fused_chunk
        chunks = [(r0, min(B, r0 + R)) for r0 in range(0, B, R)]
        C.embedding_sumsq(self.last_tokens[:B], dec.w("embed"), self.b_x[:B], ss)
        tp, Hq, Hkv = self.tp, self.Hq_l, self.Hkv_l
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            fq, fg = self._folded(i)
            wo, wd = dec.w(p + "wo"), dec.w(p + "wd")
            if tp is None:
                bq = dec.w(p + "bqkv") if cfg.attention_bias else None
            else:  # this rank's input columns of the row-parallel projections (strided views of the full matrices)
                bq = self.bq_local[i] if cfg.attention_bias else None
                wo = wo[:, self.tp_rank * self.qd_l:(self.tp_rank + 1) * self.qd_l]
                wd = wd[:, self.tp_rank * self.F_l:(self.tp_rank + 1) * self.F_l]
            for r0, r1 in chunks:
                x, x1, qkv, attn, act = (self.b_x[r0:r1], self.b_x1[r0:r1], self.b_qkv[r0:r1], self.b_attn[r0:r1], self.b_act[r0:r1])
                bt, sl = self.block_tables[r0:r1], self.seq_lens[r0:r1]
                s0, s1, s2 = ss[2 * i, r0:r1], ss[2 * i + 1, r0:r1], ss[2 * i + 2, r0:r1]
                # up to 128 rows: rotary embedding and the KV-cache write happen in the qkv GEMM's epilogue
                ok = (r1 - r0) <= 128 and C.gemm_decode_rope(x, fq, qkv, bq, s0, eps, cos_t, sin_t, bt, sl, self._kc(i), self._vc(i),
                                                             Hq, Hkv, st)
                if not ok:
                    ok = C.gemm_decode(x, fq, qkv, bq, None, s0, None, eps, st)
                    C.rope_kv_write_decode(qkv, cos_t, sin_t, bt, sl, self._kc(i), self._vc(i), Hq, Hkv, cfg.head_dim, st)
                C.paged_decode_attn(qkv, self._kc(i), self._vc(i), bt, sl, attn, Hq, Hkv,
                                    cfg.head_dim, scale, splits, self.b_part_o, self.b_part_ml, st, self.b_tickets)
                if tp is None:
                    ok = C.gemm_decode(attn, wo, x1, None, x, None, s1, eps, st) and ok
                    C.gemm_swiglu(x1, fg, act, s1, eps, st)
                    ok = C.gemm_decode(act, wd, x, None, x1, None, s2, eps, st) and ok
                else:
                    # row-parallel projections: partial product into this rank's symmetric buffer, then every member sums
                    # all partials (peer loads) + residual and accumulates the next norm's row statistic
                    ok = C.gemm_decode(attn, wo, tp.partial(0, r1 - r0), None, None, None, None, eps, st) and ok
                    tp.allreduce_residual(0, x, x1, s1)
                    C.gemm_swiglu(x1, fg, act, s1, eps, st)
                    ok = C.gemm_decode(act, wd, tp.partial(1, r1 - r0), None, None, None, None, eps, st) and ok
                    tp.allreduce_residual(1, x1, x, s2)
                if not ok:
                    raise RuntimeError("fused decode step: a GEMM shape is not served by the split-K kernel")
        h = self.b_h[:B]
        C.rmsnorm_fwd(self.b_x[:B], dec.w("final_norm"), h, None, eps)
        wl = self.layout.view(self.params, self.layout.lm_head_name())
        C.lm_sample(h, wl, temperature, self.step_seeds, self.b_sample_f, self.b_sample_i, self.b_tokens, self.b_lp, st)
        self._feed_back(B)

    def _decode_forward_mega(self, B: int, temperature: float, splits: int) -> None:
        """Embedding + statistics, ONE launch for all decoder layers, final norm, lm_head + sampling."""
        cfg, C, dec = self.cfg, self.C, self.dec
        cos_t, sin_t = dec.rope_tables(1)
        eps, st, ms = cfg.rms_norm_eps, self.status, self.mega_strides
        H, F, Q = cfg.hidden_size, cfg.intermediate_size, cfg.qkv_dim
        per = (Q + 2 * F) * H
        fq, fg = self._folded(0)
        C.embedding_sumsq(self.last_tokens[:B], dec.w("embed"), self.b_x[:B], self.b_ss)
        C.decode_layers(cfg.num_hidden_layers, B, fq, per, dec.w("layers.0.wo"), ms["wo"], fg, per, dec.w("layers.0.wd"), ms["wd"],
                        dec.w("layers.0.bqkv") if cfg.attention_bias else None, ms.get("bqkv", 0), self.b_x, self.b_x1, self.b_qkv,
                        self.b_attn, self.b_act, self.b_ss, eps, cos_t, sin_t, self.block_tables, self.seq_lens, self.cache,
                        cfg.num_attention_heads, cfg.num_key_value_heads, 1.0 / math.sqrt(cfg.head_dim), splits, self.b_part_o,
                        self.b_part_ml, self.b_tickets, self.b_partials, self.b_counters, st, self.mega_trace, self.mega_trace_layer)
        h = self.b_h[:B]
        C.rmsnorm_fwd(self.b_x[:B], dec.w("final_norm"), h, None, eps)
        wl = self.layout.view(self.params, self.layout.lm_head_name())
        C.lm_sample(h, wl, temperature, self.step_seeds, self.b_sample_f, self.b_sample_i, self.b_tokens, self.b_lp, st)
        self._feed_back(B)

    def _launch_count_decode(self, splits: int, B: int = 0) -> int:
        if self.mega_rows and 0 < B <= self.mega_rows:
            return 1 + 1 + 3
        fused = self.fused_decode and 0 < B <= self.fused_rows
        if fused:
            n_chunks = (B + self.fused_chunk - 1) // self.fused_chunk
            last = B - (n_chunks - 1) * self.fused_chunk
            per_layer = (n_chunks - 1) * (5 if self.fused_chunk <= 128 else 6) + (5 if last <= 128 else 6)
        else:
            per_layer = 9
        return 1 + per_layer * self.cfg.num_hidden_layers + 3

    def _decode(self, plan: Dict[str, Any]) -> None:
        rows = int(plan["batch_rows"])
        if rows == 0:
            return
        t_begin = time.perf_counter()
        B = min(self.max_seqs, (rows + 31) // 32 * 32)  # one captured graph per row count rounded to a warp of rows
        active = plan["active_slots"]  # int32 array of slots
        S = self.max_seqs
        ri = self.step_count % len(self.stage_ring)
        t_w = time.perf_counter()
        self.stage_events[ri].synchronize()  # the copy that last read this staging buffer has completed
        self.t_wait += time.perf_counter() - t_w
        self.h_lens[active] += 1
        self.step_count += 1
        st = self.stage_np[ri]
        st[:S] = self.h_lens
        n_upd = len(plan["upd_slot"])
        st[S] = n_upd
        st[S + 1] = (self.step_count * 0x632BE5AB) & 0x7FFFFFFF
        if n_upd:
            st[S + 4: S + 4 + n_upd] = plan["upd_slot"] * self.max_blocks_per_seq + plan["upd_index"]
            st[S + 4 + S: S + 4 + S + n_upd] = plan["upd_block"]
        self.d_stage.copy_(self.stage_ring[ri], non_blocking=True)
        self.stage_events[ri].record()
        self.h2d_bytes += self.d_stage.numel() * 4
        # lengths, positions, seeds and the new block-table entries reach their device buffers in one launch
        self.C.decode_step_inputs(self.d_stage, S, self.seq_lens, self.positions, self.block_tables, self.base_seeds,
                                  self.step_seeds, self.status)
        max_len = int(self.h_lens[:B].max())
        if self.mega_rows and B <= self.mega_rows:
            # the persistent layer kernel works on one attention item per CTA at a time: one wave of items
            want = self.sm_count // max(1, len(active) * self.cfg.num_key_value_heads)
        else:
            want = (self.sm_count * 3) // max(1, len(active) * self.cfg.num_key_value_heads)
        splits = int(max(1, min(self.max_splits, want, max(1, max_len // 256))))
        temperature = float(self.temperature or 0.0)
        t_mid = time.perf_counter()
        self.t_prep += t_mid - t_begin
        if self.use_cuda_graph:
            key = (B, temperature, splits, self.record_logprobs)
            g = self.graphs.get(key)
            if g is None:
                # Warm up outside capture (sets function attributes, fills tensor-map caches), then put back what the
                # warm-up step changed so that the captured step starts from the same state.
                keep_tok, keep_gen = self.last_tokens.clone(), self.gen_index.clone()
                self._decode_forward(B, temperature, splits)
                torch.cuda.synchronize(self.dev)
                self.last_tokens.copy_(keep_tok)
                self.gen_index.copy_(keep_gen)
                g = torch.cuda.CUDAGraph()
                # thread-local capture: the trainer / logprob threads keep allocating while this thread captures
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    self._decode_forward(B, temperature, splits)
                self.graphs[key] = g
            g.replay()
        else:
            self._decode_forward(B, temperature, splits)
        self.t_launch += time.perf_counter() - t_mid
        self.launches += self._launch_count_decode(splits, B)
        self.tokens_generated += len(active)
        self.h_gen[active] += 1
        # asynchronous token read-back for EOS detection (one step of lag), only while some sequence stops at EOS
        ring = self.step_count & 1
        if self.n_watch > 0:
            self.h_tok_pin[ring].copy_(self.b_tokens, non_blocking=True)
            self.d2h_bytes += self.max_seqs * 4
            self.tok_events[ring].record()
            # (slots, the sequence ids living in them, index of the token this step produced)
            self.tok_pending[ring] = (active.copy(), self.h_seq[active].copy(), self.h_gen[active] - 1)
        else:
            self.tok_pending[ring] = None

    def _check_lagged_eos(self, ring: int) -> None:
        pend = self.tok_pending[ring]
        if pend is None:
            return
        self.tok_events[ring].synchronize()
        slots, seqs, gen_at = pend
        toks = self.h_tok_pin[ring].numpy()
        hit = (toks[slots] == self.eos) & self.h_watch[slots] & (self.h_seq[slots] == seqs) & (self.h_eos_at[slots] < 0)
        if hit.any():
            self.h_eos_at[slots[hit]] = gen_at[hit]
        self.tok_pending[ring] = None

    def _collect_finished(self, force_eos_check: bool) -> List[FinishedSequence]:
        out: List[FinishedSequence] = []
        done = np.nonzero((self.h_seq >= 0) & ((self.h_eos_at >= 0) | (self.h_gen >= self.h_limit)))[0]
        if done.size == 0:
            return out
        done_slots = []
        for slot in done.tolist():
            info = self.slot_info[slot]
            if self.h_eos_at[slot] >= 0:
                done_slots.append((slot, info, int(self.h_eos_at[slot]) + 1, "stop"))
            else:
                done_slots.append((slot, info, int(self.h_limit[slot]), "length"))
        idx = torch.tensor([d[0] for d in done_slots], dtype=torch.int64, device=self.dev)
        width = max(d[2] for d in done_slots)
        rows = self.history[:, :width].index_select(0, idx).cpu().numpy()
        self.d2h_bytes += rows.nbytes
        lp_rows = None
        if self.record_logprobs:
            lp_rows = self.history_lp[:, :width].index_select(0, idx).cpu().numpy()
            self.d2h_bytes += lp_rows.nbytes
        for j, (slot, info, n_out, reason) in enumerate(done_slots):
            r = info["req"]
            ids = rows[j, :n_out].astype(np.int32).copy()
            if info["forced"] is not None:
                ids[-1] = self.eos  # EOS forced at the drawn length
                reason = "stop"
            out.append(FinishedSequence(r.request_id, info["child"], ids, reason, len(r.prompt),
                                        lp_rows[j, :n_out].astype(np.float32).copy() if lp_rows is not None else None))
            self.sched.finish(info["seq_id"])
            self._free_slot(slot)
        return out

    def _compact(self) -> None:
        """Moves the per-slot state of the sequences the scheduler relocates (device rows and host mirrors)."""
        for ring in (0, 1):  # pending EOS read-backs refer to the old slots: settle them first
            self._check_lagged_eos(ring)
        moves = self.sched.compact_slots()
        if not moves:
            return
        self.n_compactions += 1
        frm = np.asarray([m[0] for m in moves], dtype=np.int64)
        to = np.asarray([m[1] for m in moves], dtype=np.int64)
        idx = torch.from_numpy(np.stack([frm, to])).pin_memory().to(self.dev, non_blocking=True)
        self.h2d_bytes += idx.numel() * 8
        moved = [self.block_tables, self.last_tokens, self.gen_index, self.base_seeds, self.history]
        if self.record_logprobs:
            moved.append(self.history_lp)
        for t in moved:
            t.index_copy_(0, idx[1], t.index_select(0, idx[0]))
        self.launches += 10
        for a, empty in ((self.h_lens, 0), (self.h_gen, 0), (self.h_seq, -1), (self.h_limit, 1 << 60), (self.h_watch, False),
                         (self.h_eos_at, -1)):
            a[to] = a[frm]
            a[frm] = empty
        for f, t_ in moves:
            self.slot_info[t_] = self.slot_info.pop(f)

    def _free_slot(self, slot: int) -> None:
        self.n_watch -= int(self.h_watch[slot])
        self.h_lens[slot] = 0
        self.h_gen[slot] = 0
        self.h_seq[slot] = -1
        self.h_limit[slot] = 1 << 60
        self.h_watch[slot] = False
        self.h_eos_at[slot] = -1
        del self.slot_info[slot]

    # ------------------------------------------------------------------ stepping
    def step(self) -> List[FinishedSequence]:
        pc = time.perf_counter
        t0 = pc()
        self._admit_pending()
        did = False
        if self.sched.num_waiting > 0 and self.sched.num_free_slots > 0:
            plan = self.sched.plan_prefill()
            if plan["group_ids"]:
                self._prefill(plan)
                did = True
                self.n_prefill_steps += 1
                self.t_prefill += pc() - t0
        if not did and self.sched.num_running > 0:
            # sequences finish at different times and leave holes; when closing them saves at least 32 rows, move the
            # sequences from the highest slots down (decided from the previous step's plan)
            if self.compact_slots and (self._last_rows + 31) // 32 > (self._last_active + 31) // 32:
                self._compact()
            plan = self.sched.plan_decode()
            self._last_rows, self._last_active = int(plan["batch_rows"]), int(plan["num_active"])
            if plan["preempted"]:
                self._requeue_preempted(plan["preempted"])
            t1 = pc()
            self.t_plan += t1 - t0
            # EOS results of the previous step are examined while this step runs
            self._decode(plan)
            t2 = pc()
            self._check_lagged_eos((self.step_count - 1) & 1)
            out = self._collect_finished(False)
            self.t_post += pc() - t2
            self.n_decode_steps += 1
            return out
        return self._collect_finished(False)

    def timing_stats(self) -> Dict[str, float]:
        """Host seconds spent per phase of the step loop since construction (planning, staging, launch, bookkeeping)."""
        return {"engine_decode_steps": float(self.n_decode_steps), "engine_prefill_steps": float(self.n_prefill_steps),
                "engine_plan_s": self.t_plan, "engine_prep_s": self.t_prep, "engine_launch_s": self.t_launch,
                "engine_post_s": self.t_post, "engine_prefill_s": self.t_prefill, "engine_wait_s": self.t_wait,
                "engine_compactions": float(self.n_compactions), "engine_prefix_hit_tokens": float(self.prefix_hit_tokens),
                "engine_prefix_lookup_tokens": float(self.prefix_lookup_tokens)}

    def _requeue_preempted(self, seq_ids: List[int]) -> None:
        # A preempted sample restarts from its prompt with the same seed stream (its progress is dropped).
        for slot, info in list(self.slot_info.items()):
            if info["seq_id"] in seq_ids:
                r: _Request = info["req"]
                forced = [info["forced"]] if info["forced"] is not None else None
                self.pending.append(_Request(r.request_id, r.prompt, 1, r.max_new_tokens, r.temperature, r.seed, forced,
                                             r.ignore_eos, child_map=[info["child"]]))
                self._free_slot(slot)

    def run_until_done(self) -> List[FinishedSequence]:
        out: List[FinishedSequence] = []
        while self.has_work():
            out.extend(self.step())
        # drain the last lagged EOS check
        for ring in (0, 1):
            self._check_lagged_eos(ring)
        out.extend(self._collect_finished(True))
        return out

    def check_status(self) -> None:
        self.dec.check_status()
        if self.tp is not None:
            self.tp.check()

    def update_weights_done(self) -> None:
        """Called after new weights were written into ``params`` in place; captured graphs stay valid
        because they reference the same buffers. The norm-folded copies of the fused decode path are refreshed
        here, and the caller's stream is drained so that the engine thread's next step sees them."""
        self.sched.clear_prefix_cache()  # cached keys and values belong to the previous weights
        if self.fused_decode:
            self.refold_weights()
            torch.cuda.current_stream(self.dev).synchronize()


# =====================================================================================================
class OracleEngine:
    """Same interface, plain PyTorch, full recompute per step. For tiny models on CPU and as a test oracle."""

    def __init__(self, cfg: ModelConfig, layout: ParamLayout, params: torch.Tensor, *, max_seqs: int = 64,
                 max_model_len: Optional[int] = None, eos_token_id: Optional[int] = None, **_: Any):
        self.cfg, self.layout, self.params = cfg, layout, params
        self.dec = OracleDecoder(cfg, layout, params)
        self.max_model_len = int(max_model_len or cfg.max_position_embeddings)
        self.eos = cfg.eos_token_id if eos_token_id is None else int(eos_token_id)
        self.pending: List[_Request] = []
        self.max_seqs = max_seqs
        self.tokens_generated = 0
        self.launches = 0

    def add_request(self, request_id: Any, prompt_ids: Sequence[int], n: int = 1, max_new_tokens: int = 128,
                    temperature: float = 1.0, seed: int = 0, forced_new_tokens: Optional[Sequence[int]] = None,
                    ignore_eos: bool = False) -> None:
        prompt = np.ascontiguousarray(np.asarray(prompt_ids, dtype=np.int32))
        room = self.max_model_len - len(prompt) - 1
        max_new = max(1, min(int(max_new_tokens), room))
        forced = [max(1, min(int(f), max_new)) for f in forced_new_tokens] if forced_new_tokens is not None else None
        self.pending.append(_Request(request_id, prompt, int(n), max_new, float(temperature), int(seed), forced,
                                     bool(ignore_eos or forced is not None)))

    def has_work(self) -> bool:
        return bool(self.pending)

    @torch.no_grad()
    def _generate_group(self, r: _Request) -> List[FinishedSequence]:
        dev = self.params.device
        seqs = [list(map(int, r.prompt)) for _ in range(r.n)]
        lps: List[List[float]] = [[] for _ in range(r.n)]
        done: List[Optional[str]] = [None] * r.n
        gens = [torch.Generator(device="cpu").manual_seed(_mix_seed(r.seed, c) & 0x7FFFFFFF) for c in range(r.n)]
        wl = self.layout.view(self.params, self.layout.lm_head_name())
        for _ in range(r.max_new_tokens):
            live = [c for c in range(r.n) if done[c] is None]
            if not live:
                break
            ids = torch.tensor(sum((seqs[c] for c in live), []), dtype=torch.int32, device=dev)
            pos = torch.tensor(sum((list(range(len(seqs[c]))) for c in live), []), dtype=torch.int32, device=dev)
            cu = [0]
            for c in live:
                cu.append(cu[-1] + len(seqs[c]))
            hn = self.dec.hidden(ids, pos, cu)
            last = torch.tensor([x - 1 for x in cu[1:]], dtype=torch.long, device=dev)
            z = hn[last].float() @ wl.float().t()
            for j, c in enumerate(live):
                if r.temperature <= 0:
                    tok = int(z[j].argmax())
                    lps[c].append(float(torch.log_softmax(z[j], -1)[tok]))
                else:
                    p = torch.softmax(z[j] / r.temperature, -1).cpu()
                    tok = int(torch.multinomial(p, 1, generator=gens[c]))
                    lps[c].append(float(torch.log(p[tok])))
                seqs[c].append(tok)
                self.tokens_generated += 1
                n_new = len(seqs[c]) - len(r.prompt)
                limit = r.forced_new_tokens[c] if r.forced_new_tokens else r.max_new_tokens
                if not r.ignore_eos and tok == self.eos:
                    done[c] = "stop"
                elif n_new >= limit:
                    done[c] = "length"
        out = []
        for c in range(r.n):
            ids = np.asarray(seqs[c][len(r.prompt):], dtype=np.int32)
            reason = done[c] or "length"
            if r.forced_new_tokens:
                ids[-1] = self.eos
                reason = "stop"
            out.append(FinishedSequence(r.request_id, c, ids, reason, len(r.prompt), np.asarray(lps[c], dtype=np.float32)))
        return out

    def step(self) -> List[FinishedSequence]:
        if not self.pending:
            return []
        return self._generate_group(self.pending.pop(0))

    def run_until_done(self) -> List[FinishedSequence]:
        out: List[FinishedSequence] = []
        while self.has_work():
            out.extend(self.step())
        return out

    def check_status(self) -> None:
        return

    def update_weights_done(self) -> None:
        return
