"""Request batching, host logic only (no GPU): which waiting requests the queue stacks into one run.
Follows the reference's rule that a merged net is the concatenation of every external input along its
first dimension (blaze/blaze/scheduler/batching.cc:131-166): that is only meaningful when the requests'
per-sample inputs keep the same proportions (same candidates per user row)."""
import pkg


def api():
    pkg.load()
    from x_deeplearning_b200 import blaze_api
    return blaze_api


def test_requests_with_the_same_proportions_run_together():
    a = api()
    # [user rows, candidate rows]
    assert a.plan_batch([[1, 1000], [2, 2000], [1, 1000], [3, 3000]], 8) == [0, 1, 2, 3]


def test_other_proportions_wait_for_a_later_batch_and_order_is_kept():
    a = api()
    assert a.plan_batch([[1, 1000], [1, 500], [2, 2000], [1, 77], [4, 4000]], 8) == [0, 2, 4]
    # the head decides: with the 500-candidate request first, only its kind is picked
    assert a.plan_batch([[1, 500], [1, 1000], [2, 1000]], 8) == [0, 2]


def test_batch_size_limit_and_empty_queue():
    a = api()
    assert a.plan_batch([[1, 10]] * 5, 3) == [0, 1, 2]
    assert a.plan_batch([[1, 10]] * 5, 1) == [0]
    assert a.plan_batch([], 4) == []


def test_empty_requests_only_join_empty_heads():
    a = api()
    assert a.plan_batch([[1, 10], [0, 0], [2, 20]], 8) == [0, 2]
    assert a.plan_batch([[0, 0], [0, 0], [1, 10]], 8) == [0, 1]


def test_init_scheduler_checks_its_arguments():
    a = api()
    a.init_scheduler(False)
    try:
        a.init_scheduler(True, max_batch_size=0)
    except a.BlazeError as e:
        assert "max_batch_size" in str(e)
    else:
        raise AssertionError("max_batch_size = 0 was accepted")
    a.init_scheduler(False)


def test_host_library_exports_every_declared_entry_point():
    import ctypes
    import os
    import re
    a = api()
    header = os.path.join(os.path.dirname(a.LIB_PATH), "..", "host", "include", "blaze", "api", "c_api", "c_api_predictor.h")
    text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(Blaze_[A-Za-z0-9_]+)\s*\(", text)))
    assert len(names) >= 30
    L = ctypes.CDLL(a.LIB_PATH)
    for n in names:
        assert hasattr(L, n), "libblaze_b200.so does not export %s" % n
