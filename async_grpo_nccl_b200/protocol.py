"""Messages and data contracts shared by the roles.

``MessageType`` / ``Message`` are the trainer protocol of the reference
(gpu_process_worker.py:53-61): ``MICROBATCH(list[sample])`` -> forward/backward,
``GRADIENT_STEP`` -> clip + optimizer step, ``BATCH_DONE(aggregated metrics)`` -> completion payload.

A *sample* is a plain dict (the reference's contract, vllm_worker.py:749-796). Token arrays travel as
NumPy int32 / float32 arrays rather than Python lists:

  after generation : input_len, output_len, output_token_ids, sample_ids (prompt + output),
                     sample_position_ids, labels (-100 on the prompt, un-shifted ids on the output),
                     truncated_sample, num_non_masked_output_tokens, modified_reward, delimiter_not_found,
                     input / input_token_ids / answer (copied from the dataset row), __uid__
  after the verifier: reward, reward_success (+ adapter extras)
  after the group   : advantage, max_reward_in_group
  after logprob     : sample_logprobs, sample_entropies  (length len(sample_ids), on the logit-position
                      grid: entry p-1 is the logprob of token p)
  before training   : total_non_masked_output_tokens (sum over the ready minibatch buffer)
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Any, Dict, Optional

import numpy as np

IGNORE_INDEX = -100


class MessageType(enum.IntEnum):
    MICROBATCH = 0
    GRADIENT_STEP = 1
    BATCH_DONE = 2
    SHUTDOWN = 3


@dataclass
class Message:
    type: MessageType
    data: Any = None

    def to_wire(self) -> Dict[str, Any]:
        return {"type": int(self.type), "data": self.data}

    @staticmethod
    def from_wire(d: Dict[str, Any]) -> "Message":
        return Message(MessageType(int(d["type"])), d.get("data"))


DUMMY_TRAIN_SAMPLE: Dict[str, Any] = {"dummy": True, "total_non_masked_output_tokens": 0}


def build_sample(row: Dict[str, Any], prompt_ids: np.ndarray, output_ids: np.ndarray, eos_token_id: int,
                 text: Optional[str] = None) -> Dict[str, Any]:
    """Per-sample fields produced by the generation role (vllm_worker.py:752-774)."""
    prompt_ids = np.asarray(prompt_ids, dtype=np.int32)
    output_ids = np.asarray(output_ids, dtype=np.int32)
    sample_ids = np.concatenate([prompt_ids, output_ids])
    labels = np.concatenate([np.full(len(prompt_ids), IGNORE_INDEX, np.int32), output_ids])
    s = dict(row)
    s.update(
        input_len=int(len(prompt_ids)),
        output_token_ids=output_ids,
        output_len=int(len(output_ids)),
        sample_ids=sample_ids,
        sample_text=text if text is not None else "",
        sample_position_ids=np.arange(len(sample_ids), dtype=np.int32),
        truncated_sample=bool(len(output_ids) == 0 or int(output_ids[-1]) != int(eos_token_id)),
        labels=labels,
        num_non_masked_output_tokens=int(len(output_ids)),
        modified_reward=None,
        delimiter_not_found=False,
    )
    return s


def sample_token_count(sample: Dict[str, Any]) -> int:
    return int(sample.get("input_len", 0)) + int(sample.get("output_len", 0))


class RoleLostError(RuntimeError):
    """A role process (trainer, logprob or rollout rank) stopped answering. Raised by the orchestrator after it has
    written ``training_state.json``; the run is restarted with ``resume_state`` / ``resume_from_path`` (the reference's
    recovery path as well: it has no elastic restart, orchestrator.py:921-956)."""
