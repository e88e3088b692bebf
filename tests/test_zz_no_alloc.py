"""The allocation-free C entry point (csrc/include/agrpo_noalloc.h), called through its exported symbol.

Embedders that cannot allocate device memory at call time (all HBM already handed to a KV pool, or a serving loop
that must avoid cudaMalloc's device-wide synchronisation) call this symbol with their own input / output buffers;
the kernel's intermediate data lives in an 8 MiB array inside the library. The test loads the shared object with
ctypes, calls the symbol twice in a row on different inputs (the scratch array is shared and keeps old contents,
so the second call must not be disturbed by the first) and compares with the regular entry point. It also checks
that an oversized problem is refused. This file sorts last on purpose: a run that stops at the first failure has
then already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

OK, E_BAD_ARGUMENT, E_TOO_LARGE = 0, -1, -2


def _symbol():
    from async_grpo_nccl_b200 import _build
    from async_grpo_nccl_b200.ops import native

    native()  # makes sure the library (and libtorch, which it links against) is loaded
    lib = ctypes.CDLL(str(_build.SO_PATH))
    fn = lib.agrpo_lmhead_logprob_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return fn


def _call(fn, h, W, labels, temp, logp, ent, lse):
    msg = ctypes.create_string_buffer(512)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(h.data_ptr(), h.stride(0), W.data_ptr(), W.stride(0), labels.data_ptr(), h.shape[0], h.shape[1], W.shape[0],
            ctypes.c_float(temp), logp.data_ptr(), ent.data_ptr(), lse.data_ptr(), ctypes.c_void_p(stream), msg, 512)
    return rc, msg.value.decode()


def _reference(h, W, labels, temp):
    from async_grpo_nccl_b200.ops import native

    C = native()
    T, V = h.shape[0], W.shape[0]
    groups = C.lmhead_num_groups(V, T)
    partials = torch.empty(3 * groups * T, device="cuda")
    ll = torch.zeros(T, device="cuda")
    logp, ent, lse = (torch.empty(T, device="cuda") for _ in range(3))
    C.lmhead_logprob(h, W, labels, temp, partials, ll, logp, ent, lse, None)
    return logp, ent, lse


def test_no_alloc_entry_point_matches_regular_path_twice_in_a_row():
    fn = _symbol()
    torch.manual_seed(0)
    cases = [(700, 512, 9000, 1.0), (333, 256, 5000, 0.7)]
    inputs = []
    for T, H, V, temp in cases:
        h = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        W = (torch.randn(V, H, device="cuda") * 0.05).to(torch.bfloat16)
        labels = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
        labels[torch.rand(T, device="cuda") < 0.25] = -100
        inputs.append((h, W, labels, temp))
    outs = []
    for h, W, labels, temp in inputs:  # two calls back to back on the same stream, no synchronisation in between
        T = h.shape[0]
        logp, ent, lse = (torch.full((T,), 123.0, device="cuda") for _ in range(3))
        rc, msg = _call(fn, h, W, labels, temp, logp, ent, lse)
        assert rc == OK, msg
        outs.append((logp, ent, lse))
    torch.cuda.synchronize()
    # the status word of the kernels behind the entry point: 0 = no bounded wait ran out, the outputs are valid
    import ctypes as _ct

    from async_grpo_nccl_b200 import _build as _b

    lib = _ct.CDLL(str(_b.SO_PATH))
    lib.agrpo_lmhead_noalloc_status.restype = _ct.c_int
    lib.agrpo_lmhead_noalloc_status.argtypes = [_ct.c_void_p]
    assert lib.agrpo_lmhead_noalloc_status(_ct.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    for (h, W, labels, temp), (logp, ent, lse) in zip(inputs, outs):
        r_logp, r_ent, r_lse = _reference(h, W, labels, temp)
        torch.cuda.synchronize()
        # same kernels, same reduction order: the tolerance of the kernel tests is far looser than what is seen here
        assert (logp - r_logp).abs().max().item() < 2e-2
        assert (ent - r_ent).abs().max().item() < 2e-2
        assert (lse - r_lse).abs().max().item() < 2e-2
        assert torch.equal(logp, r_logp) and torch.equal(lse, r_lse)
        assert (logp[labels < 0] == 0).all()
        # and against plain PyTorch
        z = h.float() @ W.float().t() / temp
        want = (z.gather(1, labels.clamp(min=0).long()[:, None])[:, 0] - torch.logsumexp(z, -1)) * (labels >= 0)
        assert (logp - want).abs().max().item() < 2e-2


def test_no_alloc_entry_point_rejects_what_does_not_fit():
    fn = _symbol()
    T, H, V = 32768, 64, 152064  # (3 * groups + 1) * T * 4 bytes = 15 MB, beyond the built-in 8 MiB
    h = torch.zeros(T, H, device="cuda", dtype=torch.bfloat16)
    W = torch.zeros(8, H, device="cuda", dtype=torch.bfloat16)  # never read: the call is refused before any launch
    labels = torch.zeros(T, device="cuda", dtype=torch.int32)
    out = torch.zeros(T, device="cuda")
    msg = ctypes.create_string_buffer(512)
    rc = fn(h.data_ptr(), H, W.data_ptr(), H, labels.data_ptr(), T, H, V, ctypes.c_float(1.0), out.data_ptr(), None, None, None,
            msg, 512)
    assert rc == E_TOO_LARGE and b"too large" in msg.value
    rc = fn(h.data_ptr(), H, W.data_ptr(), H, labels.data_ptr(), 128, 60, 1000, ctypes.c_float(1.0), out.data_ptr(), None, None,
            None, msg, 512)
    assert rc == E_BAD_ARGUMENT
    torch.cuda.synchronize()
