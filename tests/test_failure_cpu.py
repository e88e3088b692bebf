"""Failure handling among CPU ranks (gloo + RPC): a role process that leaves between macro-batches, and control
messages that arrive late. Nothing here touches a GPU."""
import asyncio
import json
import os
import time

import numpy as np
import pytest

from async_grpo_nccl_b200.data import synthetic_prompt_rows


def _entry(rank, world, port, cfg_dict, rows, flag_dir, leaver, q):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port)})
    from async_grpo_nccl_b200.config import make_config
    from async_grpo_nccl_b200.launch import DistributedRuntime
    from async_grpo_nccl_b200.orchestrator import Orchestrator, configure_logging, stamp_uids
    from async_grpo_nccl_b200.protocol import RoleLostError

    configure_logging()
    cfg = make_config(cfg_dict)
    rt = DistributedRuntime(cfg)
    flag = os.path.join(flag_dir, "first_batch_done")
    if rank == leaver:
        # serves its role until rank 0 reports the first macro-batch (incl. weight sync) complete, then the process
        # exits: no kernel or collective of this rank is in flight at that point
        async def serve_then_leave():
            await rt._start_server()
            while not os.path.exists(flag):
                await asyncio.sleep(0.05)
            os._exit(0)

        asyncio.run(serve_then_leave())
        return
    if rank != 0:
        rt.serve_forever()
        return
    orch = Orchestrator(cfg, runtime=rt, dataset=rows)

    async def body():
        await rt.initialize(orch)
        em = rt.experience_manager
        for r in rt.trainer_ranks:
            em.register_training_process(r, cfg.max_tokens_per_gpu, cfg.train_minibatch_sample_size)
        await rt.start_trainers()
        data = stamp_uids(rows)
        bs = cfg.batch_size
        rec = await orch._run_macro_batch(data[:bs], 0)
        await orch.save_checkpoint()
        open(flag, "w").write("1")
        await asyncio.sleep(1.0)  # the leaver is gone by now
        t0 = time.time()
        try:
            await orch._run_macro_batch(data[bs:2 * bs], 0)
            out = ("no error", 0.0)
        except RoleLostError as e:
            out = ("RoleLostError", time.time() - t0, str(e))
        except Exception as e:  # any other exception type is a test failure
            out = (type(e).__name__, time.time() - t0, str(e))
        q.put({"first_samples": int(rec["training/batch_total_samples"]), "second": out, "global_step": orch.global_step})
        await rt.shutdown()

    asyncio.run(body())
    os._exit(0)  # the gloo group has a dead member: do not wait in its destructor


@pytest.mark.timeout(600)
@pytest.mark.parametrize("leaver,role", [(2, "generation"), (1, "logprob")])
def test_role_process_leaving_between_macro_batches_is_noticed_and_state_is_resumable(tmp_path, leaver, role):
    import torch.multiprocessing as mp

    from async_grpo_nccl_b200 import checkpoint as ckpt

    cfg = dict(model_name_or_path="tiny", batch_size=4, samples_per_question=2, num_epochs=1, train_minibatch_sample_size=8,
               max_generation_tokens=8, max_tokens_per_gpu=400, reward_fns=["token_match"], global_num_verifiers=0,
               num_training_gpu_workers=1, num_logprob_gpu_workers=1, num_generation_gpu_workers=1,
               placement={"trainer": [0], "logprob": [1], "rollout": [2]}, learning_rate=1e-3, output_dir=str(tmp_path / "out"),
               min_samples_per_checkpoint=10 ** 9, eval_at_start=False, stream_logprobs=False, trainer_completion_timeout_s=20.0,
               prompt_timeout_s=30.0)
    rows = synthetic_prompt_rows(8, 1024, 16, 32, seed=0)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29783 + leaver
    procs = [ctx.Process(target=_entry, args=(r, 3, port, cfg, rows, str(tmp_path), leaver, q)) for r in range(3)]
    for p in procs:
        p.start()
    try:
        res = q.get(timeout=400)
    finally:
        for p in procs:
            p.join(timeout=20)
        for p in procs:
            if p.is_alive():
                p.kill()
    assert res["first_samples"] == 8
    kind, seconds, msg = res["second"]
    assert kind == "RoleLostError", res["second"]
    assert role in msg and seconds < 60.0, (msg, seconds)
    # what a restart needs is on disk: the counters of the last completed macro-batch and its checkpoint
    st = json.load(open(tmp_path / "out" / "training_state.json"))
    assert st["global_step"] == 1 and st["macro_batch_count"] == 1 and st["total_samples_seen"] == 8
    path = ckpt.latest_checkpoint(str(tmp_path / "out"))
    assert path is not None and ckpt.load_scheduler_state(path)["opt_step"] == 1
    assert os.path.exists(os.path.join(path, "config.json"))


def test_delayed_control_messages_do_not_lose_or_reorder_results():
    """RPC calls whose handlers answer late and out of order: every caller still gets its own answer; a call whose answer
    is later than its timeout raises instead of waiting forever."""
    from async_grpo_nccl_b200.rpc import RpcClient, RpcServer

    class Slow:
        async def echo(self, i, delay):
            await asyncio.sleep(delay)
            return {"i": i, "payload": np.arange(i, dtype=np.int32)}

    async def body():
        srv = RpcServer(Slow(), "127.0.0.1", 0)
        port = await srv.start()
        cli = await RpcClient("127.0.0.1", port, name="slow").connect()
        delays = [0.30, 0.05, 0.20, 0.0, 0.10]
        res = await asyncio.gather(*[cli.call("echo", i, d) for i, d in enumerate(delays)])
        assert [r["i"] for r in res] == list(range(5))
        assert all(len(r["payload"]) == i for i, r in enumerate(res))
        with pytest.raises(asyncio.TimeoutError):
            await cli.call("echo", 9, 1.0, timeout=0.1)
        assert (await cli.call("echo", 3, 0.0))["i"] == 3  # the connection is still usable after a timed-out call
        await cli.close()
        await srv.close()

    asyncio.run(body())
