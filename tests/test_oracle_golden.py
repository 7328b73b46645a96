"""Pins the CPU oracle against the reference's own operator fixtures and, for
pooling, against the reference sparse store compiled unmodified."""
import json
import os

import numpy as np
import pytest

import orc
import oracle_net

HERE = os.path.dirname(os.path.abspath(__file__))
FIX = json.load(open(os.path.join(HERE, "golden", "blaze_op_fixtures.json")))
SKIP = {"sparse_op/embedding/embedding_v1.conf"}  # needs the mock puller: covered in test_embedding_op


@pytest.mark.parametrize("name", sorted(k for k in FIX if k not in SKIP))
def test_oracle_matches_reference_fixture(name):
    net = FIX[name]
    env = oracle_net.run_net(net)
    assert net["expected"], "fixture without expectation"
    for out, exp in net["expected"].items():
        got = np.asarray(env[out], dtype=np.float64)
        want = np.array(exp["values"], dtype=np.float64).reshape(exp["shape"])
        assert list(got.shape) == list(exp["shape"]), (got.shape, exp["shape"])
        # the reference harness accepts |d| <= 1e-6 or 5 % relative
        # (blaze/blaze/test/operator/operator_test_common.h:66-76); the fixtures
        # print ~7 significant digits, so 2e-6 + 1e-5 relative is the tight bar here.
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=2e-6)
