"""llmcp_dev_gated_delta_net_noalloc against llmcp_op_gated_delta_net.

The no-allocation entry point serves hosts that cannot call cudaMalloc while they run (a
process that has given the whole GPU to its own memory pool, a decode loop that cannot absorb
an allocation's synchronisation).  Its working memory is one array inside the library shared by
all calls, so the test makes two calls in a row with different inputs: the second must not be
disturbed by what the first left in the array.  Outputs and the updated recurrent state have to
be bit-identical to the allocating entry point's and to the CPU oracle's.  This file is collected
last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

import llmcp_b200 as L
import oracle

pytestmark = pytest.mark.gpu


def _inputs(rng, S, nk, nv, dk, dv):
    channels = 2 * nk * dk + nv * dv
    bf16 = lambda a: (np.asarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)
    return dict(conv=bf16(rng.standard_normal((S, channels))), a=bf16(rng.standard_normal((S, nv))),
                b=bf16(rng.standard_normal((S, nv))), a_log=(rng.standard_normal(nv) * 0.2).astype(np.float32),
                dt_bias=bf16(rng.standard_normal(nv) * 0.2),
                state=(rng.standard_normal((nv, dk, dv)) * 0.1).astype(np.float32))


def _upload(torch, x, S, nv, dv):
    dev = {k: torch.from_numpy(v.view(np.int16) if v.dtype == np.uint16 else v).cuda() for k, v in x.items()}
    return dev, torch.empty((S, nv * dv), dtype=torch.int16, device="cuda")


def _call(torch, dev, out, S, nk, nv, dk, dv):
    ptr = lambda t: C.c_void_p(t.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    rc = L.lib().llmcp_dev_gated_delta_net_noalloc(
        ptr(dev["conv"]), ptr(dev["a"]), ptr(dev["b"]), ptr(dev["a_log"]), ptr(dev["dt_bias"]), ptr(dev["state"]),
        C.c_int64(S), C.c_int64(nk), C.c_int64(nv), C.c_int64(dk), C.c_int64(dv), 0, ptr(out), C.c_void_p(stream))
    torch.cuda.synchronize()
    return rc


def _noalloc(torch, x, S, nk, nv, dk, dv):
    dev, out = _upload(torch, x, S, nv, dv)
    rc = _call(torch, dev, out, S, nk, nv, dk, dv)
    return rc, out.cpu().numpy().view(np.uint16), dev["state"].cpu().numpy()


def test_noalloc_matches_allocating_entry_point_twice():
    torch = pytest.importorskip("torch")
    torch.cuda.set_device(0)
    L.set_device(0)
    rng = np.random.default_rng(2026)
    # decode shape of the model, then a short multi-token call: different sizes back to back
    for S, nk, nv, dk, dv in ((1, 16, 32, 128, 128), (7, 16, 32, 128, 128)):
        x = _inputs(rng, S, nk, nv, dk, dv)
        want_out, want_state = L.ops.gated_delta_net(x["conv"], x["a"], x["b"], x["a_log"], x["dt_bias"], x["state"],
                                                     nk, nv, dk, dv)
        rc, out, state = _noalloc(torch, x, S, nk, nv, dk, dv)
        assert rc == 0, L.last_error()
        assert np.array_equal(out, want_out)
        assert np.array_equal(state.view(np.uint32), want_state.view(np.uint32))
        # and against the CPU oracle directly, not only through the allocating entry point
        oracle_out, oracle_state = oracle.gated_delta_net(x["conv"], x["a"], x["b"], x["a_log"], x["dt_bias"], x["state"],
                                                          nk, nv, dk, dv)
        assert np.array_equal(out, oracle_out)
        assert np.array_equal(state.view(np.uint32), oracle_state.view(np.uint32))


def test_noalloc_leaves_free_device_memory_unchanged():
    """After one call per kernel (one token, several tokens) further calls take no device memory: the
    free byte count of the GPU is the same before and after them (inputs and output are uploaded
    before the first reading, so nothing else allocates in between)."""
    torch = pytest.importorskip("torch")
    torch.cuda.set_device(0)
    L.set_device(0)
    rng = np.random.default_rng(3)
    shapes = ((1, 16, 32, 128, 128), (7, 16, 32, 128, 128))
    held = []
    for S, nk, nv, dk, dv in shapes:
        dev, out = _upload(torch, _inputs(rng, S, nk, nv, dk, dv), S, nv, dv)
        assert _call(torch, dev, out, S, nk, nv, dk, dv) == 0, L.last_error()  # the start-up call of this kernel
        held.append((dev, out))
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        for (S, nk, nv, dk, dv), (dev, out) in zip(shapes, held):
            assert _call(torch, dev, out, S, nk, nv, dk, dv) == 0
    assert torch.cuda.mem_get_info()[0] == free_before


def test_noalloc_rejects_oversized_calls():
    torch = pytest.importorskip("torch")
    torch.cuda.set_device(0)
    rng = np.random.default_rng(1)
    S, nk, nv, dk, dv = 16, 16, 32, 128, 128  # 16 * 4160 floats > 65536
    x = _inputs(rng, S, nk, nv, dk, dv)
    rc, _, state = _noalloc(torch, x, S, nk, nv, dk, dv)
    assert rc == 2 and "65536" in L.last_error()
    assert np.array_equal(state, x["state"])  # nothing ran
    L.lib().llmcp_b200_clear_error()
