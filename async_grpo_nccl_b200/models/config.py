"""Decoder architecture description (Qwen2 / Qwen2.5 / Llama-3 style dense decoders).

The reference loads whatever ``AutoModelForCausalLM`` returns for ``model_name_or_path``
(gpu_process_worker.py:652-657) and assumes a Qwen2 decoder layer for FSDP wrapping
(gpu_process_worker.py:33, 407-411). Here the architecture is an explicit record that can be read
from an HF ``config.json`` or given inline for random-init runs.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional


@dataclass(frozen=True)
class ModelConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    attention_bias: bool = True  # Qwen2: q/k/v projections carry a bias; Llama: none
    model_type: str = "qwen2"
    eos_token_id: int = 0
    bos_token_id: Optional[int] = None
    initializer_range: float = 0.02

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def num_parameters(self) -> int:
        h, f, v = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = 2 * h + self.qkv_dim * h + (self.qkv_dim if self.attention_bias else 0) + h * self.q_dim + 3 * h * f
        n = v * h + self.num_hidden_layers * per_layer + h
        if not self.tie_word_embeddings:
            n += v * h
        return n

    def to_hf_dict(self) -> Dict[str, Any]:
        arch = "Qwen2ForCausalLM" if self.model_type == "qwen2" else "LlamaForCausalLM"
        d = {
            "architectures": [arch],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "torch_dtype": "bfloat16",
            "eos_token_id": self.eos_token_id,
            "initializer_range": self.initializer_range,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.model_type == "llama":
            d["attention_bias"] = self.attention_bias
        return d

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "ModelConfig":
        if "preset" in d:
            base = PRESETS[d["preset"]].to_dict()
            base.update({k: v for k, v in d.items() if k != "preset"})
            d = base
        model_type = d.get("model_type", "qwen2")
        heads = int(d["num_attention_heads"])
        hidden = int(d["hidden_size"])
        eos = d.get("eos_token_id", 0)
        if isinstance(eos, (list, tuple)):
            eos = eos[0]
        return ModelConfig(
            vocab_size=int(d["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(d["intermediate_size"]),
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=heads,
            num_key_value_heads=int(d.get("num_key_value_heads", heads)),
            head_dim=int(d.get("head_dim") or hidden // heads),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_theta=float(d.get("rope_theta", 1e6 if model_type == "qwen2" else 5e5)),
            max_position_embeddings=int(d.get("max_position_embeddings", 32768)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", model_type == "qwen2")),
            model_type=model_type,
            eos_token_id=int(eos if eos is not None else 0),
            bos_token_id=d.get("bos_token_id"),
            initializer_range=float(d.get("initializer_range", 0.02)),
        )

    @staticmethod
    def from_pretrained(path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as f:
            return ModelConfig.from_dict(json.load(f))


PRESETS: Dict[str, ModelConfig] = {
    # CPU / gloo plumbing model
    "tiny": ModelConfig(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e4,
                        max_position_embeddings=2048, tie_word_embeddings=False, eos_token_id=1),
    # same shape family with head_dim 128 so that every GPU kernel path is exercised on a small model
    "tiny128": ModelConfig(vocab_size=2048, hidden_size=512, intermediate_size=1408, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=128, rope_theta=1e4,
                           max_position_embeddings=4096, tie_word_embeddings=True, eos_token_id=1),
    "qwen2.5-1.5b": ModelConfig(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                                num_attention_heads=12, num_key_value_heads=2, head_dim=128, rope_theta=1e6,
                                max_position_embeddings=32768, tie_word_embeddings=True, eos_token_id=151643),
    "qwen2.5-7b": ModelConfig(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                              num_attention_heads=28, num_key_value_heads=4, head_dim=128, rope_theta=1e6,
                              max_position_embeddings=32768, tie_word_embeddings=False, eos_token_id=151643),
    "qwen2.5-32b": ModelConfig(vocab_size=152064, hidden_size=5120, intermediate_size=27648, num_hidden_layers=64,
                               num_attention_heads=40, num_key_value_heads=8, head_dim=128, rope_theta=1e6,
                               max_position_embeddings=32768, tie_word_embeddings=False, eos_token_id=151643),
    "llama-3-70b": ModelConfig(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                               num_attention_heads=64, num_key_value_heads=8, head_dim=128, rope_theta=5e5,
                               max_position_embeddings=8192, tie_word_embeddings=False, attention_bias=False,
                               model_type="llama", eos_token_id=128001),
}


def resolve_model_config(model_name_or_path: Optional[str], inline: Optional[Dict[str, Any]]) -> ModelConfig:
    """Inline dict wins; otherwise a preset name or a directory holding ``config.json``."""
    if inline:
        return ModelConfig.from_dict(inline)
    if model_name_or_path in PRESETS:
        return PRESETS[model_name_or_path]
    if model_name_or_path and os.path.isdir(model_name_or_path):
        return ModelConfig.from_pretrained(model_name_or_path)
    raise FileNotFoundError(f"cannot resolve model config from {model_name_or_path!r}")
