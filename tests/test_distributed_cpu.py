"""The full role graph as separate processes over gloo + RPC on CPU: 2 trainer ranks (sharded optimizer state),
1 rank hosting logprob + rollout. Checks that collectives line up, that both trainer ranks end with the same
parameters and that the weight sync delivered them to the inference rank."""
import numpy as np
import pytest

from async_grpo_nccl_b200.data import synthetic_prompt_rows
from async_grpo_nccl_b200.launch import spawn


@pytest.mark.timeout(600)
def test_three_process_pipeline(tmp_path):
    cfg = dict(model_name_or_path="tiny", batch_size=4, samples_per_question=4, num_epochs=1, train_minibatch_sample_size=8,
               max_generation_tokens=10, max_tokens_per_gpu=200, reward_fns=["token_match"], global_num_verifiers=0,
               num_training_gpu_workers=2, num_logprob_gpu_workers=1, num_generation_gpu_workers=1,
               placement={"trainer": [0, 1], "logprob": [2], "rollout": [2]}, learning_rate=1e-3, output_dir=str(tmp_path),
               min_samples_per_checkpoint=10 ** 9, eval_at_start=False, verify_weight_sync_during_init=True)
    rows = synthetic_prompt_rows(8, 1024, 16, 32, seed=0)
    out = spawn(cfg, rows, world=3, max_macro_batches=2, port=29711, timeout_s=500)
    assert out["global_step"] == 2
    assert out["total_samples_seen"] == 32
    last = out["last"]
    assert last["training/optimizer_steps_in_batch"] == 2
    assert np.isfinite(last["training/avg_loss"]) and last["training/grad_norm"] > 0
