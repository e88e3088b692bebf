"""Checkpoint / resume in the reference's directory layout.

``output_dir/hf_format/step_<global_step>_samples_<total>/`` holds an HF-loadable model
(``model-0000k-of-0000n.safetensors`` + ``model.safetensors.index.json`` or a single
``model.safetensors``, ``config.json``, tokenizer files when available), the optimizer state and
``scheduler_state.pt``; ``output_dir/training_state.json`` holds the orchestrator counters
(gpu_process_worker.py:1081-1223, orchestrator.py:263-300, 1389-1434).

Differences: tensors are written with HF names straight from the flat layout (fused qkv / gate_up are
split into row ranges, no state-dict gather through Python objects); optimizer state is one safetensors
file per trainer rank plus a manifest, and is re-sharded on load when the trainer world size changed.
"""
from __future__ import annotations

import json
import os
import re
import shutil
from typing import Any, Dict, List, Optional, Tuple

import torch

from .models.config import ModelConfig
from .models.layout import ParamLayout

_CKPT_RE = re.compile(r"step_(\d+)_samples_(\d+)$")


def checkpoint_dir(output_dir: str, global_step: int, total_samples: int) -> str:
    return os.path.join(output_dir, "hf_format", f"step_{global_step}_samples_{total_samples}")


# ---- model weights -------------------------------------------------------------------------------
def save_hf_model(path: str, cfg: ModelConfig, layout: ParamLayout, flat: torch.Tensor, max_shard_bytes: int = 5 << 30,
                  tokenizer_src: Optional[str] = None) -> List[str]:
    """Writes bf16 safetensors shards with HF tensor names. ``flat`` is the full flat parameter buffer."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for name, t in layout.hf_items(flat):
        tb = t.detach().to(torch.bfloat16).cpu().contiguous()
        nbytes = tb.numel() * 2
        if size + nbytes > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][name] = tb
        size += nbytes
    files: List[str] = []
    if len(shards) == 1:
        fn = "model.safetensors"
        save_file(shards[0], os.path.join(path, fn), metadata={"format": "pt"})
        files.append(fn)
    else:
        weight_map: Dict[str, str] = {}
        total = 0
        for i, sh in enumerate(shards):
            fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file(sh, os.path.join(path, fn), metadata={"format": "pt"})
            files.append(fn)
            for k, v in sh.items():
                weight_map[k] = fn
                total += v.numel() * 2
        with open(os.path.join(path, "model.safetensors.index.json"), "w", encoding="utf-8") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg.to_hf_dict(), f, indent=2)
    if tokenizer_src and os.path.isdir(tokenizer_src):
        for fn in os.listdir(tokenizer_src):
            if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "special_tokens_map.json", "added_tokens.json",
                                                    "generation_config.json"):
                shutil.copy2(os.path.join(tokenizer_src, fn), os.path.join(path, fn))
    return files


def load_hf_model(path: str, layout: ParamLayout, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reads an HF checkpoint directory into a flat fp32 buffer laid out by ``layout``."""
    from safetensors import safe_open

    if out is None:
        out = torch.zeros(layout.total, dtype=torch.float32)
    files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors") and not f.startswith("optimizer"))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {path}")
    dest = dict(layout.hf_items(out))
    seen = set()
    for fn in files:
        with safe_open(os.path.join(path, fn), framework="pt", device="cpu") as f:
            for key in f.keys():
                if key not in dest:
                    if key == "lm_head.weight" and layout.cfg.tie_word_embeddings:
                        continue
                    raise KeyError(f"unexpected tensor {key} in {fn}")
                t = f.get_tensor(key)
                if tuple(t.shape) != tuple(dest[key].shape):
                    raise ValueError(f"shape mismatch for {key}: {tuple(t.shape)} vs {tuple(dest[key].shape)}")
                dest[key].copy_(t.to(torch.float32))
                seen.add(key)
    missing = [k for k in dest if k not in seen]
    if missing:
        raise KeyError(f"checkpoint is missing {len(missing)} tensors, e.g. {missing[:3]}")
    return out


# ---- optimizer / scheduler ---------------------------------------------------------------------------
def save_optimizer_shard(path: str, rank: int, world: int, layout: ParamLayout, state: Dict[str, torch.Tensor],
                         scheduler: Dict[str, Any]) -> None:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    save_file({k: v.detach().cpu().contiguous() for k, v in state.items()},
              os.path.join(path, f"optimizer-rank{rank:05d}-of-{world:05d}.safetensors"))
    if rank == 0:
        with open(os.path.join(path, "optimizer_manifest.json"), "w", encoding="utf-8") as f:
            json.dump({"world": world, "total": layout.total, "num_units": len(layout.unit_ranges),
                       "shard_numel": layout.shard_numel()}, f)
        torch.save(scheduler, os.path.join(path, "scheduler_state.pt"))


def load_optimizer_shard(path: str, rank: int, world: int, layout: ParamLayout) -> Optional[Dict[str, torch.Tensor]]:
    """Returns this rank's {master, exp_avg, exp_avg_sq}; re-shards when the saved world size differs."""
    from safetensors.torch import load_file

    man_path = os.path.join(path, "optimizer_manifest.json")
    if not os.path.exists(man_path):
        return None
    with open(man_path, "r", encoding="utf-8") as f:
        man = json.load(f)
    saved_world = int(man["world"])
    if saved_world == world:
        return load_file(os.path.join(path, f"optimizer-rank{rank:05d}-of-{world:05d}.safetensors"))
    # rebuild full flat tensors from the saved shards, then cut this rank's shard
    old_layout = ParamLayout(layout.cfg, shard_world=saved_world)
    keys = ("master", "exp_avg", "exp_avg_sq")
    full = {k: torch.zeros(max(old_layout.total, layout.total), dtype=torch.float32) for k in keys}
    for r in range(saved_world):
        sh = load_file(os.path.join(path, f"optimizer-rank{r:05d}-of-{saved_world:05d}.safetensors"))
        for lo, gs, ln in old_layout.local_to_global_ranges(r):
            for k in keys:
                # unit padding may differ between layouts; copy segment by segment
                full[k][gs:gs + ln] = sh[k][lo:lo + ln]
    if old_layout.total != layout.total:
        # padding differs: move every named segment to its new offset
        moved = {k: torch.zeros(layout.total, dtype=torch.float32) for k in keys}
        for name, seg in layout.segments.items():
            oseg = old_layout.segments[name]
            for k in keys:
                moved[k][seg.offset:seg.offset + seg.numel] = full[k][oseg.offset:oseg.offset + oseg.numel]
        full = moved
    out = {k: torch.empty(layout.shard_numel(), dtype=torch.float32) for k in keys}
    for lo, gs, ln in layout.local_to_global_ranges(rank):
        for k in keys:
            out[k][lo:lo + ln] = full[k][gs:gs + ln]
    return out


def load_scheduler_state(path: str) -> Optional[Dict[str, Any]]:
    p = os.path.join(path, "scheduler_state.pt")
    return torch.load(p, weights_only=False) if os.path.exists(p) else None


# ---- orchestrator counters ---------------------------------------------------------------------------
def save_training_state(output_dir: str, state: Dict[str, Any]) -> None:
    os.makedirs(output_dir, exist_ok=True)
    tmp = os.path.join(output_dir, "training_state.json.tmp")
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(state, f, indent=2)
    os.replace(tmp, os.path.join(output_dir, "training_state.json"))


def load_training_state(output_dir: str) -> Optional[Dict[str, Any]]:
    p = os.path.join(output_dir, "training_state.json")
    if not os.path.exists(p):
        return None
    with open(p, "r", encoding="utf-8") as f:
        return json.load(f)


def list_checkpoints(output_dir: str) -> List[Tuple[int, int, str]]:
    root = os.path.join(output_dir, "hf_format")
    out = []
    if os.path.isdir(root):
        for d in os.listdir(root):
            m = _CKPT_RE.search(d)
            if m:
                out.append((int(m.group(2)), int(m.group(1)), os.path.join(root, d)))
    return sorted(out)


def prune_checkpoints(output_dir: str, keep_last_n: int) -> List[str]:
    """Keeps the ``keep_last_n`` checkpoints with the most samples seen (orchestrator.py:1409-1432)."""
    ck = list_checkpoints(output_dir)
    removed = []
    for _, _, path in ck[:-keep_last_n] if keep_last_n > 0 else []:
        shutil.rmtree(path, ignore_errors=True)
        removed.append(path)
    return removed


def latest_checkpoint(output_dir: str) -> Optional[str]:
    ck = list_checkpoints(output_dir)
    return ck[-1][2] if ck else None
