"""Pins the pooling restatement (oracle.c orc_embedding_pool) against
(a) the known-answer case of the reference's own unit test
    (blaze/blaze/test/store/quick_embedding/quick_embedding_dict_test.cc:100-241) and
(b) the reference sparse store compiled from its own sources (oracle/_ref),
    on seeded random tables, when that library has been built."""
import numpy as np
import pytest

import orc

KEY1, KEY2, KEY3, KEY4 = 1032342412, 849234344343, 3434234243, 5230242044
CASE1 = np.array([[1.0, 1.0, 3.0, 1.0]], np.float32)
CASE2 = np.array([[0.15, 0.3, 2.0, 1.0, 1.0, 2.0, 0.23, 3.0]], np.float32)
CASE34 = np.array([[2.5, 1.0, 0.15, 0.3, 2.0, 1.0], [1.0, 0.15, 0.3, 2.0, 1.0, 1.0]], np.float32)


def _kat(pool):
    """pool(table_name, table_keys, weights, keys, values, key_num, items)"""
    b1 = np.full((2, 12), np.nan, np.float32)
    b2 = np.full((2, 24), np.nan, np.float32)
    pool("101", [KEY1], CASE1, [1032342412, 12312422], [2.0, 1.2], [1, 1], [dict(udf=0, out=b1, col=0)])
    pool("102", [KEY2], CASE2, [2324222, KEY2, KEY2], [2.0, 1.2, 1.0], [1, 2], [dict(udf=0, out=b1, col=4)])
    pool("104_7", [KEY3, KEY4], CASE34, [KEY3, KEY4, 2424123, KEY3, 0, KEY4], [1.0] * 6, [4, 2],
         [dict(udf=2, trunc_dir=0, trunc_num=4, out=b2, col=0)])
    np.testing.assert_allclose(b1[0, :4], CASE1[0] * 2.0, rtol=1e-6)
    assert (b1[0, 4:] == 0).all()                       # missing key -> zeros
    assert (b1[1, :4] == 0).all()
    np.testing.assert_allclose(b1[1, 4:], CASE2[0] * np.float32(2.2), rtol=1e-6)   # duplicated key
    want = np.zeros((2, 24), np.float32)
    want[0, 0:6], want[0, 6:12], want[0, 18:24] = CASE34[0], CASE34[1], CASE34[0]
    want[1, 6:12] = CASE34[1]
    np.testing.assert_array_equal(b2, want)


def test_oracle_known_answer():
    def pool(name, tkeys, w, keys, values, key_num, items):
        orc.embedding_pool(w, keys, values, key_num, items, table_keys=tkeys)
    _kat(pool)


needs_ref = pytest.mark.skipif(orc.ref_lib() is None, reason="oracle/_ref not built")


@needs_ref
def test_reference_store_known_answer(tmp_path):
    st = orc.RefStore({"101": ([KEY1], CASE1), "102": ([KEY2], CASE2), "104_7": ([KEY3, KEY4], CASE34)},
                      str(tmp_path / "kat.qed"))

    def pool(name, tkeys, w, keys, values, key_num, items):
        assert st.get(name, keys, values, key_num, items) == 0
    _kat(pool)
    st.close()


@needs_ref
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_oracle_equals_reference_store(tmp_path, seed):
    rng = np.random.default_rng(seed)
    rows, dim, batch = 5000, [4, 16, 18][seed], 64
    tkeys = rng.choice(1 << 40, size=rows, replace=False).astype(np.int64)
    w = rng.normal(0, 0.01, (rows, dim)).astype(np.float32)
    st = orc.RefStore({"t": (tkeys, w)}, str(tmp_path / "r.qed"))
    key_num = rng.integers(0, 12, batch).astype(np.int32)          # includes empty samples
    n = int(key_num.sum())
    keys = tkeys[rng.integers(0, rows, n)]
    miss = rng.random(n) < 0.1
    keys[miss] = rng.integers(1 << 41, 1 << 42, miss.sum())          # keys that are not in the table
    values = rng.normal(1, 0.5, n).astype(np.float32)
    tn = 5
    width = dim + dim + dim * tn + dim * tn

    def items(out):
        return [dict(udf=0, out=out, col=0), dict(udf=1, out=out, col=dim),
                dict(udf=2, trunc_dir=0, trunc_num=tn, out=out, col=2 * dim),
                dict(udf=2, trunc_dir=1, trunc_num=tn, out=out, col=2 * dim + dim * tn)]
    a = np.full((batch, width), 7.0, np.float32)
    b = np.full((batch, width), 7.0, np.float32)
    assert st.get("t", keys, values, key_num, items(a)) == 0
    orc.embedding_pool(w, keys, values, key_num, items(b), table_keys=tkeys)
    np.testing.assert_array_equal(a, b)                               # same order of fp32 operations
    assert st.get("absent_table", keys, values, key_num, items(a)) == 0   # table miss: kOK, untouched
    st.close()
