"""Bounded waits: a wait that can never be satisfied gives up after its limit, the device status word says
where, and the context stays usable (no trap, no fault, no hang: the kernel simply returns)."""
import numpy as np
import pytest
import torch

import orc
import pkg

pytestmark = pytest.mark.gpu


def test_wait_runs_out_sets_status_and_context_survives():
    pkg.load()
    from x_deeplearning_b200 import capi, ops
    L = capi.lib()
    assert ops.device_status() == 0
    capi.check(L.xb_selftest_wait_timeout(200_000, ops.stream()))          # about 0.1 ms
    torch.cuda.synchronize()
    st = ops.device_status()
    assert st != 0 and (st >> 8) == 99 and (st & 0xff) == 1, st
    # sticky until cleared
    assert ops.device_status() == st
    capi.check(L.xb_device_status_clear())
    assert ops.device_status() == 0
    # the context is intact: a tensor-core GEMM right after gives the right answer
    rng = np.random.default_rng(0)
    A = rng.normal(0, 1, (256, 64)).astype(np.float16)
    W = rng.normal(0, 0.2, (64, 32)).astype(np.float16)
    Wk = ops.pack_weight_kmajor(torch.from_numpy(W).cuda(), torch.float16)
    Y = ops.gemm(torch.from_numpy(A).cuda(), Wk, trans_b=True, M=256, N=32, K=64, engine=capi.XB_GEMM_TCGEN05)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    want = orc.gemm_op(A.astype(np.float32), W.astype(np.float32))
    np.testing.assert_allclose(Y.float().cpu().numpy(), want, rtol=2e-3, atol=2e-3)


def test_predictor_forward_fails_after_a_wait_ran_out_and_recovers():
    """The host runtime reads the status word after every run: a Forward whose stream saw a bounded wait give
    up returns false with the site in the error text, clears the word, and the next Forward succeeds."""
    pkg.load()
    from x_deeplearning_b200 import blaze_api as api, capi, ops
    L = capi.lib()
    text = api.netdef_text([api.op_text("Sigmoid", ["x"], ["y"], {})], [("x", 1)], [("y", 1)])
    mgr = api.PredictorManager()
    mgr.load_model_text(text)
    p = mgr.create_predictor()
    x = np.linspace(-2, 2, 64).astype(np.float32).reshape(8, 8)
    keep = p.feed("x", x)
    p.forward()
    capi.check(L.xb_selftest_wait_timeout(200_000, None))      # legacy stream: ordered before the next run
    torch.cuda.synchronize()
    with pytest.raises(Exception, match="bounded wait ran out.*site 99"):
        p.forward()
    assert ops.device_status() == 0                              # cleared by the runtime
    p.forward()
    np.testing.assert_allclose(p.output("y"), 1 / (1 + np.exp(-x)), rtol=1e-6, atol=1e-6)
    p.close()
    mgr.close()


def test_status_mirror_is_a_host_word():
    pkg.load()
    import ctypes as C
    from x_deeplearning_b200 import capi, ops
    L = capi.lib()
    word = C.POINTER(C.c_int32)()
    capi.check(L.xb_device_status_mirror(C.byref(word)))
    again = C.POINTER(C.c_int32)()
    capi.check(L.xb_device_status_mirror(C.byref(again)))
    assert C.addressof(word.contents) == C.addressof(again.contents)
    assert word[0] == 0
    capi.check(L.xb_selftest_wait_timeout(200_000, ops.stream()))
    torch.cuda.synchronize()
    assert word[0] == (99 << 8 | 1) == ops.device_status()
    capi.check(L.xb_device_status_clear())
    assert word[0] == 0 and ops.device_status() == 0


def test_wait_selftest_rejects_bad_limit():
    pkg.load()
    from x_deeplearning_b200 import capi, ops
    with pytest.raises(capi.XbError, match="limit of"):
        capi.check(capi.lib().xb_selftest_wait_timeout(0, ops.stream()))
