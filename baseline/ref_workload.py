"""Synthetic workload of the headline benchmark for the reference arm (no import from ``async_grpo_nccl_b200``).

Same rows as ``async_grpo_nccl_b200.data.synthetic_prompt_rows`` (a CPU test compares the two generators
element for element), the same Bernoulli reward, and a model directory that ``from_pretrained`` and vLLM can
load offline: ``config.json`` of the named architecture, random-init bf16 safetensors and a minimal tokenizer.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Any, Dict, List, Sequence

import numpy as np

ARCHS: Dict[str, Dict[str, Any]] = {
    "qwen2.5-1.5b": dict(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                         num_attention_heads=12, num_key_value_heads=2, rope_theta=1e6, max_position_embeddings=32768,
                         tie_word_embeddings=True, eos_token_id=151643, rms_norm_eps=1e-6),
    "qwen2.5-7b": dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                       num_attention_heads=28, num_key_value_heads=4, rope_theta=1e6, max_position_embeddings=32768,
                       tie_word_embeddings=False, eos_token_id=151643, rms_norm_eps=1e-6),
    "tiny128": dict(vocab_size=2048, hidden_size=512, intermediate_size=1408, num_hidden_layers=2,
                    num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4, max_position_embeddings=4096,
                    tie_word_embeddings=True, eos_token_id=1, rms_norm_eps=1e-6),
}


def synthetic_rows(num_prompts: int, vocab_size: int, min_len: int, max_len: int, seed: int, samples_per_question: int,
                   gen_len_range: Sequence[int], reward_p: float) -> List[Dict[str, Any]]:
    rng = np.random.default_rng(seed)
    rows = []
    for i in range(num_prompts):
        L = int(rng.integers(min_len, max_len + 1))
        ids = rng.integers(0, vocab_size, L, dtype=np.int64).astype(np.int32)
        lo, hi = int(gen_len_range[0]), int(gen_len_range[1])
        lens = np.exp(rng.uniform(math.log(lo), math.log(hi), samples_per_question))
        rows.append({"input_token_ids": ids, "input": "", "answer": "", "__uid__": i,
                     "forced_output_lens": [int(max(1, round(float(x)))) for x in lens], "reward_p": float(reward_p)})
    return rows


def bernoulli_reward(sample: Dict[str, Any], p: float = 0.3) -> float:
    ids = np.asarray(sample["input_token_ids"], dtype=np.int64)
    h = hashlib.sha256(ids[: int(sample["input_len"])].tobytes())
    h.update(np.asarray(sample.get("output_token_ids", []), dtype=np.int64)[:8].tobytes())
    h.update(str(sample.get("sample_index", 0)).encode())
    u = int.from_bytes(h.digest()[:8], "little") / float(1 << 64)
    return float(u < float(sample.get("reward_p", p)))


def build_model_dir(path: str, arch: str, seed: int = 0) -> str:
    """Writes config.json, random-init bf16 weights (HF initialisation, N(0, 0.02)) and a tokenizer; idempotent."""
    done = os.path.join(path, ".complete")
    if os.path.exists(done):
        return path
    os.makedirs(path, exist_ok=True)
    import torch
    from transformers import Qwen2Config, Qwen2ForCausalLM

    a = ARCHS[arch]
    cfg = Qwen2Config(**a, hidden_act="silu", torch_dtype="bfloat16", bos_token_id=a["eos_token_id"],
                      pad_token_id=a["eos_token_id"], initializer_range=0.02, use_cache=True,
                      max_window_layers=a["num_hidden_layers"], use_sliding_window=False)
    torch.manual_seed(seed)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = Qwen2ForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    model.save_pretrained(path, safe_serialization=True)
    del model
    if dev == "cuda":
        torch.cuda.empty_cache()
    _write_tokenizer(path, a["vocab_size"], a["eos_token_id"])
    with open(done, "w") as f:
        f.write("ok\n")
    return path


def _write_tokenizer(path: str, vocab_size: int, eos_id: int) -> None:
    """A word-level tokenizer with one token per id (``AutoTokenizer.from_pretrained`` needs files to load)."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit
    from transformers import PreTrainedTokenizerFast

    vocab = {f"t{i}": i for i in range(vocab_size)}
    eos = f"t{eos_id}"
    tok = Tokenizer(WordLevel(vocab, unk_token=eos))
    tok.pre_tokenizer = WhitespaceSplit()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, eos_token=eos, pad_token=eos, bos_token=eos, unk_token=eos)
    fast.save_pretrained(path)
    cfg_path = os.path.join(path, "tokenizer_config.json")
    with open(cfg_path) as f:
        tc = json.load(f)
    tc["tokenizer_class"] = "PreTrainedTokenizerFast"
    with open(cfg_path, "w") as f:
        json.dump(tc, f)
