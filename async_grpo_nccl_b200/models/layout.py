"""One canonical flat parameter layout shared by the trainer, logprob and rollout roles.

All parameters live in one flat buffer: unit 0 holds the embedding table, the final norm and (when
untied) the lm_head; unit ``1 + i`` holds decoder layer ``i`` with the q/k/v projections fused into
one ``wqkv`` matrix and gate/up fused into ``wgu``. Every tensor starts on a 256-byte boundary and
every unit is padded so it splits evenly over the sharding world size. Because all roles use the same
layout, the trainer -> rollout/logprob weight sync is a cast plus a copy of contiguous ranges: no key
conversion and no per-tensor ``load_weights`` as in the reference (gpu_process_worker.py:421-439,
1904-1913). HF tensor names exist only at the checkpoint boundary (``hf_items``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, List, Tuple

import torch

from .config import ModelConfig

ALIGN = 128  # elements


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass(frozen=True)
class Segment:
    name: str  # e.g. "layers.3.wqkv"
    offset: int  # element offset in the flat buffer
    shape: Tuple[int, ...]
    unit: int

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class ParamLayout:
    def __init__(self, cfg: ModelConfig, shard_world: int = 1):
        self.cfg = cfg
        self.shard_world = max(1, int(shard_world))
        self.segments: Dict[str, Segment] = {}
        self.unit_ranges: List[Tuple[int, int]] = []  # [start, end) element range of each unit (padded)
        off = 0
        pad_to = ALIGN * self.shard_world

        def add(name: str, shape: Tuple[int, ...], unit: int) -> None:
            nonlocal off
            seg = Segment(name, off, shape, unit)
            self.segments[name] = seg
            off = _round_up(off + seg.numel, ALIGN)

        h, f, v = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
        start = off
        add("embed", (v, h), 0)
        add("final_norm", (h,), 0)
        if not cfg.tie_word_embeddings:
            add("lm_head", (v, h), 0)
        off = _round_up(off, pad_to)
        self.unit_ranges.append((start, off))
        for i in range(cfg.num_hidden_layers):
            start = off
            u = i + 1
            add(f"layers.{i}.ln1", (h,), u)
            add(f"layers.{i}.wqkv", (cfg.qkv_dim, h), u)
            if cfg.attention_bias:
                add(f"layers.{i}.bqkv", (cfg.qkv_dim,), u)
            add(f"layers.{i}.wo", (h, cfg.q_dim), u)
            add(f"layers.{i}.ln2", (h,), u)
            add(f"layers.{i}.wgu", (2 * f, h), u)
            add(f"layers.{i}.wd", (h, f), u)
            off = _round_up(off, pad_to)
            self.unit_ranges.append((start, off))
        self.total = off

    # ---- views ----
    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        seg = self.segments[name]
        return flat[seg.offset: seg.offset + seg.numel].view(seg.shape)

    def lm_head_name(self) -> str:
        return "embed" if self.cfg.tie_word_embeddings else "lm_head"

    def shard_range(self, unit: int, rank: int) -> Tuple[int, int]:
        """Element range of ``unit`` owned by ``rank`` under even sharding."""
        s, e = self.unit_ranges[unit]
        n = (e - s) // self.shard_world
        return s + rank * n, s + (rank + 1) * n

    def shard_numel(self) -> int:
        return self.total // self.shard_world

    def local_to_global_ranges(self, rank: int) -> List[Tuple[int, int, int]]:
        """(local_offset, global_start, length) triples mapping a rank's contiguous shard buffer to the flat buffer."""
        out = []
        lo = 0
        for u in range(len(self.unit_ranges)):
            s, e = self.shard_range(u, rank)
            out.append((lo, s, e - s))
            lo += e - s
        return out

    # ---- init ----
    def init_random_(self, flat: torch.Tensor, seed: int = 0) -> None:
        """N(0, initializer_range) weights, unit norm scales, zero biases; identical on every device."""
        gen = torch.Generator(device="cpu").manual_seed(seed)
        flat.zero_()
        std = self.cfg.initializer_range
        for name, seg in self.segments.items():
            dst = self.view(flat, name)
            leaf = name.split(".")[-1]
            if leaf in ("ln1", "ln2", "final_norm"):
                dst.fill_(1.0)
            elif leaf == "bqkv":
                dst.zero_()
            else:
                # generate in row blocks to bound host memory for large tables
                rows = seg.shape[0]
                step = max(1, (1 << 24) // max(1, seg.numel // rows))
                for r0 in range(0, rows, step):
                    r1 = min(rows, r0 + step)
                    blk = torch.randn((r1 - r0,) + tuple(seg.shape[1:]), generator=gen, dtype=torch.float32) * std
                    dst[r0:r1].copy_(blk)

    def init_random_device_(self, flat: torch.Tensor, seed: int = 0) -> None:
        """Same distribution as ``init_random_`` generated on ``flat``'s device (fast for multi-billion-parameter
        models). Ranks that pass the same seed on the same device type get identical values."""
        gen = torch.Generator(device=flat.device).manual_seed(seed)
        flat.zero_()
        std = self.cfg.initializer_range
        for name, seg in self.segments.items():
            dst = flat[seg.offset: seg.offset + seg.numel]
            leaf = name.split(".")[-1]
            if leaf in ("ln1", "ln2", "final_norm"):
                dst.fill_(1.0)
            elif leaf == "bqkv":
                dst.zero_()
            else:
                dst.normal_(0.0, std, generator=gen)

    # ---- HF checkpoint boundary ----
    def hf_items(self, flat: torch.Tensor) -> Iterator[Tuple[str, torch.Tensor]]:
        """Yield (hf_name, tensor view) pairs in HF naming; fused matrices are split into row ranges."""
        cfg = self.cfg
        yield "model.embed_tokens.weight", self.view(flat, "embed")
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            yield p + "input_layernorm.weight", self.view(flat, f"layers.{i}.ln1")
            w = self.view(flat, f"layers.{i}.wqkv")
            q, k = cfg.q_dim, cfg.kv_dim
            yield p + "self_attn.q_proj.weight", w[:q]
            yield p + "self_attn.k_proj.weight", w[q:q + k]
            yield p + "self_attn.v_proj.weight", w[q + k:]
            if cfg.attention_bias:
                b = self.view(flat, f"layers.{i}.bqkv")
                yield p + "self_attn.q_proj.bias", b[:q]
                yield p + "self_attn.k_proj.bias", b[q:q + k]
                yield p + "self_attn.v_proj.bias", b[q + k:]
            yield p + "self_attn.o_proj.weight", self.view(flat, f"layers.{i}.wo")
            yield p + "post_attention_layernorm.weight", self.view(flat, f"layers.{i}.ln2")
            gu = self.view(flat, f"layers.{i}.wgu")
            f = cfg.intermediate_size
            yield p + "mlp.gate_proj.weight", gu[:f]
            yield p + "mlp.up_proj.weight", gu[f:]
            yield p + "mlp.down_proj.weight", self.view(flat, f"layers.{i}.wd")
        yield "model.norm.weight", self.view(flat, "final_norm")
        if not cfg.tie_word_embeddings:
            yield "lm_head.weight", self.view(flat, "lm_head")

    def weights_info(self) -> List[Tuple[str, Tuple[int, ...], str]]:
        """[(hf_key, shape, dtype)] metadata, the counterpart of get_trainer_weights_info (gpu_process_worker.py:1583-1602)."""
        probe = torch.empty(0)
        out = []
        meta = torch.empty(self.total, dtype=torch.bfloat16, device="meta")
        for name, t in self.hf_items(meta):
            out.append((name, tuple(t.shape), "bfloat16"))
        del probe
        return out
