"""C++ packer against the NumPy restatement and against a direct Python oracle of the contract."""
import numpy as np
import torch

from async_grpo_nccl_b200.packing import make_dummy_batch, pack_for_logprob, pack_samples


def _samples(rng, n):
    out = []
    for i in range(n):
        li, lo = int(rng.integers(1, 200)), int(rng.integers(0, 300))
        L = li + lo
        out.append(dict(sample_ids=rng.integers(0, 1000, L).astype(np.int32), input_len=li, output_len=lo, advantage=float(i) - 1.5,
                        sample_logprobs=rng.normal(size=L).astype(np.float32), sample_entropies=rng.normal(size=L).astype(np.float32),
                        reward=float(i % 2), truncated_sample=bool(i % 3 == 0)))
    return out


def test_native_packer_equals_numpy_and_python_oracle():
    rng = np.random.default_rng(0)
    for n in (1, 2, 7):
        ss = _samples(rng, n)
        a = pack_samples(ss, pin=False, use_native=True)
        b = pack_samples(ss, pin=False, use_native=False)
        assert torch.equal(a.int_buf, b.int_buf) and torch.equal(a.float_buf, b.float_buf)
        off, oidx = 0, []
        for i, s in enumerate(ss):
            li, lo = s["input_len"], s["output_len"]
            L = li + lo
            ids = s["sample_ids"]
            assert np.array_equal(a.ids[off:off + L].numpy(), ids)
            assert np.array_equal(a.pos[off:off + L].numpy(), np.arange(L))
            for p in range(L):
                want = ids[p + 1] if (p + 1 >= li and p + 1 < L) else -100  # left-shifted labels
                assert a.labels[off + p].item() == want
            assert np.allclose(a.advantages[off:off + L].numpy(), s["advantage"])
            assert np.allclose(a.old_logprobs[off:off + L].numpy(), s["sample_logprobs"])
            assert np.allclose(a.output_lens_broadcasted[off:off + L].numpy(), lo)
            oidx += [off + li - 1 + j for j in range(lo)]
            off += L
            assert a.cu_seqlens[i + 1].item() == off
        assert a.output_indices.tolist() == oidx
        assert int((a.labels >= 0).sum()) == len(oidx)
        tiles = a.tiles.numpy()
        assert (tiles[:-1, 2] >= tiles[1:, 2]).all()  # heaviest query tile first
        assert len(tiles) == sum((len(s["sample_ids"]) + 127) // 128 for s in ss)
        assert a.tiles.data_ptr() % 16 == a.int_buf.data_ptr() % 16
        assert a.scalars["num_samples"] == n and a.scalars["num_output_tokens"] == sum(s["output_len"] for s in ss)


def test_dummy_and_logprob_packing():
    d = make_dummy_batch()
    assert d.dummy and d.T == 1 and int((d.labels >= 0).sum()) == 0
    assert pack_samples([{"dummy": True}], pin=False).dummy
    ss = _samples(np.random.default_rng(1), 3)
    lp = pack_for_logprob(ss, pin=False)
    off = 0
    for s in ss:
        L = len(s["sample_ids"])
        assert np.array_equal(lp.labels[off:off + L - 1].numpy(), s["sample_ids"][1:])
        assert lp.labels[off + L - 1].item() == -100
        off += L
