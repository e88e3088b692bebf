"""Padding-free sample packing.

``pack_samples`` turns a list of sample dicts (the contract the generation role produces, see
:mod:`async_grpo_nccl_b200.protocol`) into one ``PackedBatch``: every per-token field concatenated to
``[T]``, position ids restarting per sample, left-shifted labels, ``cu_seqlens``, the attention tile
table, ``output_indices`` and the scalar counters of the reference's ``post_process_batch``
(sample_processing_utils.py:159-223). The hot loop lives in the C++ packer (csrc/host/packer.cpp) and
writes into one pinned buffer per dtype, so ``to_device`` is two host-to-device copies per microbatch
instead of the reference's per-sample, per-field copies (gpu_process_worker.py:1672-1686).
A NumPy restatement is kept as the oracle and as the fallback where the extension is not built.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

ATTN_TILE = 128
IGNORE = -100


@dataclass
class PackedBatch:
    T: int
    n: int
    total_out: int
    n_tiles: int
    int_buf: torch.Tensor  # int32: ids | pos | labels | cu_seqlens | output_indices | tiles
    float_buf: torch.Tensor  # fp32: adv | old_logp | old_ent | ref_logp | out_len
    has_ref: bool = False
    scalars: Dict[str, float] = field(default_factory=dict)
    uids: List[Any] = field(default_factory=list)
    dummy: bool = False

    def _i(self, start: int, n: int) -> torch.Tensor:
        return self.int_buf[start:start + n]

    def _f(self, k: int) -> torch.Tensor:
        return self.float_buf[k * self.T:(k + 1) * self.T]

    @property
    def ids(self) -> torch.Tensor:
        return self._i(0, self.T)

    @property
    def pos(self) -> torch.Tensor:
        return self._i(self.T, self.T)

    @property
    def labels(self) -> torch.Tensor:
        return self._i(2 * self.T, self.T)

    @property
    def cu_seqlens(self) -> torch.Tensor:
        return self._i(3 * self.T, self.n + 1)

    @property
    def output_indices(self) -> torch.Tensor:
        return self._i(3 * self.T + self.n + 1, self.total_out)

    @property
    def tiles(self) -> torch.Tensor:
        return self._i(tiles_offset(self.T, self.n, self.total_out), 4 * self.n_tiles).view(self.n_tiles, 4)

    @property
    def advantages(self) -> torch.Tensor:
        return self._f(0)

    @property
    def old_logprobs(self) -> torch.Tensor:
        return self._f(1)

    @property
    def old_entropies(self) -> torch.Tensor:
        return self._f(2)

    @property
    def ref_logprobs(self) -> Optional[torch.Tensor]:
        return self._f(3) if self.has_ref else None

    @property
    def output_lens_broadcasted(self) -> torch.Tensor:
        return self._f(4)

    def h2d_bytes(self) -> int:
        return self.int_buf.numel() * 4 + self.float_buf.numel() * 4

    def to_device(self, device, non_blocking: bool = True) -> "PackedBatch":
        if self.int_buf.device == torch.device(device):
            return self
        ib = self.int_buf.to(device, non_blocking=non_blocking)
        fb = self.float_buf.to(device, non_blocking=non_blocking)
        return PackedBatch(self.T, self.n, self.total_out, self.n_tiles, ib, fb, self.has_ref, dict(self.scalars),
                           list(self.uids), self.dummy)


def tiles_offset(T: int, n: int, total_out: int) -> int:
    """Offset of the tile table in the int buffer, rounded up to 4 words so kernels can read it as int4."""
    return (3 * T + n + 1 + total_out + 3) // 4 * 4


def _as_i32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.int32))


def _as_f32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32))


def _gather_inputs(samples: Sequence[Dict[str, Any]]):
    ids = np.concatenate([_as_i32(s["sample_ids"]) for s in samples]) if samples else np.zeros(0, np.int32)
    in_lens = _as_i32([int(s["input_len"]) for s in samples])
    out_lens = _as_i32([int(s["output_len"]) for s in samples])
    adv = _as_f32([float(s.get("advantage", 0.0)) for s in samples])

    def per_token(key: str) -> Optional[np.ndarray]:
        if not samples or any(s.get(key) is None for s in samples):
            return None
        return np.concatenate([_as_f32(s[key]) for s in samples])

    return ids, in_lens, out_lens, adv, per_token("sample_logprobs"), per_token("sample_entropies"), per_token("ref_logprobs")


def pack_numpy(ids, in_lens, out_lens, adv, logprobs, entropies, ref_logprobs, tile: int = ATTN_TILE):
    """NumPy oracle of the C++ packer. Returns (int_buf, float_buf, n_tiles)."""
    n = len(in_lens)
    T = int(ids.shape[0])
    total_out = int(out_lens.sum()) if n else 0
    pos = np.zeros(T, np.int32)
    labels = np.full(T, IGNORE, np.int32)
    cu = np.zeros(n + 1, np.int32)
    oidx = np.zeros(total_out, np.int32)
    advb = np.zeros(T, np.float32)
    outlen = np.zeros(T, np.float32)
    tiles = []
    off = 0
    oo = 0
    for i in range(n):
        li, lo = int(in_lens[i]), int(out_lens[i])
        L = li + lo
        pos[off:off + L] = np.arange(L, dtype=np.int32)
        if lo > 0:
            # rows li-1 .. L-2 predict output tokens li .. L-1
            labels[off + li - 1: off + L - 1] = ids[off + li: off + L]
            oidx[oo:oo + lo] = off + li - 1 + np.arange(lo, dtype=np.int32)
        advb[off:off + L] = adv[i]
        outlen[off:off + L] = lo
        for q0 in range(0, L, tile):
            tiles.append((off, L, q0, 0))
        oo += lo
        off += L
        cu[i + 1] = off
    order = sorted(range(len(tiles)), key=lambda j: -tiles[j][2])  # stable: Python sort keeps ties in order
    tiles_arr = np.asarray([tiles[j] for j in order], np.int32).reshape(-1, 4) if tiles else np.zeros((0, 4), np.int32)
    zeros = np.zeros(T, np.float32)
    pad = np.zeros(tiles_offset(T, n, total_out) - (3 * T + n + 1 + total_out), np.int32)
    int_buf = np.concatenate([ids.astype(np.int32), pos, labels, cu, oidx, pad, tiles_arr.reshape(-1)])
    float_buf = np.concatenate([advb, logprobs if logprobs is not None else zeros,
                                entropies if entropies is not None else zeros,
                                ref_logprobs if ref_logprobs is not None else zeros, outlen])
    return int_buf, float_buf, len(tiles)


def make_dummy_batch(pin: bool = False) -> PackedBatch:
    """Single masked token: keeps collectives aligned on ranks that got no real sample
    (the role of the reference's make_dummy_batch, sample_processing_utils.py:127-157)."""
    pb = pack_samples([{"sample_ids": [0], "input_len": 1, "output_len": 0, "advantage": 0.0}], pin=pin)
    pb.dummy = True
    pb.scalars["num_samples"] = 0
    return pb


def pack_samples(samples: Sequence[Dict[str, Any]], pin: bool = True, use_native: Optional[bool] = None) -> PackedBatch:
    real = [s for s in samples if not s.get("dummy", False)]
    if not real:
        if samples:
            return make_dummy_batch(pin=pin)
        raise ValueError("pack_samples: empty sample list")
    ids, in_lens, out_lens, adv, lp, ent, ref = _gather_inputs(real)
    n = len(real)
    T = int(ids.shape[0])
    total_out = int(out_lens.sum())
    if use_native is None:
        from .ops import have_native

        use_native = have_native()
    pin = bool(pin and torch.cuda.is_available())
    if use_native:
        from .ops import native

        C = native()
        t_in, t_out = torch.from_numpy(in_lens), torch.from_numpy(out_lens)
        n_tiles = int(C.pack_count_tiles(t_in, t_out, ATTN_TILE))
        int_buf = torch.zeros(tiles_offset(T, n, total_out) + 4 * n_tiles, dtype=torch.int32, pin_memory=pin)
        float_buf = torch.empty(5 * T, dtype=torch.float32, pin_memory=pin)
        C.pack_microbatch(torch.from_numpy(ids), t_in, t_out, torch.from_numpy(adv),
                          torch.from_numpy(lp) if lp is not None else None,
                          torch.from_numpy(ent) if ent is not None else None,
                          torch.from_numpy(ref) if ref is not None else None, ATTN_TILE, int_buf, float_buf)
    else:
        ib, fb, n_tiles = pack_numpy(ids, in_lens, out_lens, adv, lp, ent, ref)
        int_buf, float_buf = torch.from_numpy(ib), torch.from_numpy(fb)
        if pin:
            int_buf, float_buf = int_buf.pin_memory(), float_buf.pin_memory()
    scalars = {
        "num_output_tokens_non_masked": float(sum(int(s.get("num_non_masked_output_tokens", s["output_len"])) for s in real)),
        "num_output_tokens": float(total_out),
        "num_samples": float(n),
        "max_reward_in_group": float(sum(float(s.get("max_reward_in_group", 0.0)) for s in real)),
        "total_modified_reward": float(sum(float(s.get("modified_reward") or 0.0) for s in real)),
        "total_non_modified_reward": float(sum(float(s.get("reward", 0.0)) for s in real)),
        "total_reward_rank": float(sum(float(s.get("reward", 0.0)) for s in real)),
        "delimiter_not_found": float(sum(1.0 for s in real if s.get("delimiter_not_found", False))),
        "truncated_sample": float(sum(1.0 for s in real if s.get("truncated_sample", False))),
        "total_non_masked_output_tokens": float(real[0].get("total_non_masked_output_tokens", total_out)),
        "num_tokens": float(T),
    }
    return PackedBatch(T, n, total_out, n_tiles, int_buf, float_buf, ref is not None, scalars,
                       [s.get("__uid__") for s in real])


def pack_for_logprob(samples: Sequence[Dict[str, Any]], pin: bool = True) -> PackedBatch:
    """Packing for the logprob role: every row of a sample gets a label (the next token), so logprobs come back
    on the full logit-position grid like the reference's eval-mode forward (gpu_process_worker.py:1672-1703)."""
    shadow = []
    for s in samples:
        L = len(s["sample_ids"])
        shadow.append({"sample_ids": s["sample_ids"], "input_len": 1, "output_len": L - 1, "advantage": 0.0})
    return pack_samples(shadow, pin=pin)
