"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations. numpy only; shared by the GPU path, the CPU oracle
and the parity tests so that both sides consume identical arrays.

The DIN/DIEN reference models are trained on a public product-review dump that
is not available here; these generators stand in for it (same dims: embedding 18,
item+category key 36, behaviour length 100, attention MLP 144-80-40-1, tower
324-200-80-2).
"""
import numpy as np


def zipf_ranks(rng, n_rows, size, s):
    """Ranks in [0, n_rows) with P(rank r) ~ 1/(r+1)^s. Exact inverse CDF for small
    universes, continuous power-law inverse for large ones."""
    u = rng.random(size)
    if n_rows <= 20_000_000:
        w = 1.0 / np.power(np.arange(1, n_rows + 1, dtype=np.float64), s)
        cdf = np.cumsum(w)
        cdf /= cdf[-1]
        return np.minimum(np.searchsorted(cdf, u), n_rows - 1).astype(np.int64)
    a = 1.0 - s
    r = np.power(u * (np.power(n_rows + 1.0, a) - 1.0) + 1.0, 1.0 / a) - 1.0
    return np.clip(r.astype(np.int64), 0, n_rows - 1)


def scatter_rows(ranks, n_rows):
    """Affine bijection rank -> row so that hot rows are spread over the table."""
    mult = 2654435761 % n_rows
    while np.gcd(mult, n_rows) != 1:
        mult += 1
    return (ranks * mult + 12345) % n_rows


def zipf_ids(rng, n_rows, size, s):
    return scatter_rows(zipf_ranks(rng, n_rows, size, s), n_rows).astype(np.int64)


def fp16_round(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


# ---------------------------------------------------------------------------
def embedding_config(seed=0, rows=1_000_000, dim=16, batch=512, groups=20, max_len=50, s=1.1, sigma=0.01):
    """Sum-pooling benchmark: one fp32 table, `groups` feature groups over it,
    lengths uniform in [1, max_len], Zipf ids, unit weights, CSR int32 offsets."""
    rng = np.random.default_rng(seed)
    table = rng.normal(0.0, sigma, (rows, dim)).astype(np.float32)
    out = {"table": table, "groups": []}
    for g in range(groups):
        counts = rng.integers(1, max_len + 1, batch).astype(np.int32)
        n = int(counts.sum())
        ids = zipf_ids(rng, rows, n, s)
        offsets = np.zeros(batch + 1, np.int32)
        np.cumsum(counts, out=offsets[1:])
        out["groups"].append({"ids": ids, "counts": counts, "offsets": offsets,
                              "values": np.ones(n, np.float32)})
    return out


# ---------------------------------------------------------------------------
DIN_DIMS = dict(emb=18, d=36, T=100, h0=80, h1=40, user_groups=8, tower=(200, 80, 2))


def din_model(seed=0, item_rows=5_000_000, cate_rows=10_000, user_rows=100_000, sigma=0.01, emb_sigma=None):
    """Random-init DIN-style model. All values are fp16-representable so that the
    fp16 GPU model and the fp32 CPU oracle read identical numbers."""
    rng = np.random.default_rng(seed)
    D = DIN_DIMS
    e = D["emb"]
    es = sigma if emb_sigma is None else emb_sigma
    m = {"dims": dict(D, item_rows=item_rows, cate_rows=cate_rows, user_rows=user_rows)}
    m["item"] = fp16_round(rng.normal(0, es, (item_rows, e)))
    m["cate"] = fp16_round(rng.normal(0, es, (cate_rows, e)))
    m["user"] = [fp16_round(rng.normal(0, es, (user_rows, e))) for _ in range(D["user_groups"])]

    def lin(k, n):
        return fp16_round(rng.normal(0, 1.0 / np.sqrt(k), (k, n))), fp16_round(rng.normal(0, 0.01, n))

    def dice(n):
        return (fp16_round(rng.uniform(0, 0.5, n)), fp16_round(rng.normal(0, 0.1, n)),
                fp16_round(rng.uniform(0.5, 1.5, n)))

    d = D["d"]
    m["att"] = {}
    m["att"]["W0"], m["att"]["b0"] = lin(4 * d, D["h0"])
    m["att"]["W1"], m["att"]["b1"] = lin(D["h0"], D["h1"])
    m["att"]["W2"], b2 = lin(D["h1"], 1)
    m["att"]["b2"] = b2
    m["att"]["g0"], m["att"]["m0"], m["att"]["v0"] = dice(D["h0"])
    m["att"]["g1"], m["att"]["m1"], m["att"]["v1"] = dice(D["h1"])
    tin = D["user_groups"] * e + 5 * d
    t1, t2, t3 = D["tower"]
    m["tower"] = {}
    m["tower"]["W1"], m["tower"]["b1"] = lin(tin, t1)
    m["tower"]["W2"], m["tower"]["b2"] = lin(t1, t2)
    m["tower"]["W3"], m["tower"]["b3"] = lin(t2, t3)
    m["tower"]["dice1"] = dice(t1)
    m["tower"]["dice2"] = dice(t2)
    return m


def dien_model(seed=0, **kw):
    """Random-init DIEN-style model: the DIN tables, a GRU over the behaviour rows (hidden 36), an attention
    MLP 144-80-40-1 with sigmoid activations scoring every GRU state against the candidate, an AUGRU gated
    by those scores, and a final MLP [user | q | his_sum | q*his_sum | final state] -> 200 -> 80 -> 2 with PReLU."""
    m = din_model(seed, **kw)
    rng = np.random.default_rng(seed + 7)
    D = m["dims"]
    H = D["d"]

    def w(k, n, scale=1.0):
        return fp16_round(rng.normal(0, scale / np.sqrt(k), (k, n)))
    m["gru"] = dict(i2h=w(H, 3 * H), h2h=w(H, 3 * H), i2h_bias=fp16_round(rng.normal(0, 0.05, 3 * H)),
                    h2h_bias=fp16_round(rng.normal(0, 0.05, 3 * H)))
    m["augru"] = dict(Wg=w(2 * H, 2 * H), bg=fp16_round(rng.normal(0, 0.05, 2 * H)), Wc=w(2 * H, H),
                      bc=fp16_round(rng.normal(0, 0.05, H)))
    tin = D["user_groups"] * D["emb"] + 4 * H
    t1, t2, t3 = D["tower"]
    m["dien_tower"] = dict(W1=w(tin, t1), b1=fp16_round(rng.normal(0, 0.01, t1)), W2=w(t1, t2),
                           b2=fp16_round(rng.normal(0, 0.01, t2)), W3=w(t2, t3), b3=fp16_round(rng.normal(0, 0.01, t3)),
                           slope1=fp16_round(rng.uniform(0.1, 0.4, t1)), slope2=fp16_round(rng.uniform(0.1, 0.4, t2)))
    return m


def din_requests(model, seed, requests, n_cand=1000, s=1.1, seq_len=None):
    """`requests` requests of one user and n_cand candidate items each."""
    rng = np.random.default_rng(seed)
    D = model["dims"]
    T = D["T"]
    r = {"requests": requests, "n_cand": n_cand, "T": T}
    r["user_ids"] = np.stack([zipf_ids(rng, D["user_rows"], requests, s) for _ in range(D["user_groups"])], 1)
    if seq_len is None:
        seq = np.full(requests, T, np.int32)
    else:
        seq = np.asarray(seq_len, np.int32)
    r["seq_len"] = seq
    n = int(seq.sum())
    r["hist_item"] = zipf_ids(rng, D["item_rows"], n, s)
    r["hist_cate"] = zipf_ids(rng, D["cate_rows"], n, s)
    r["cand_item"] = zipf_ids(rng, D["item_rows"], requests * n_cand, s)
    r["cand_cate"] = zipf_ids(rng, D["cate_rows"], requests * n_cand, s)
    return r


# ---------------------------------------------------------------------------
def parallel_gemm_config(seed=0, P=8, M=4096, K=256, N=128):
    """FusedParallelGemm + bias + PReLU benchmark (per-branch inputs, axis-1 concat)."""
    rng = np.random.default_rng(seed)
    return {
        "A": fp16_round(rng.normal(0, 1, (P, M, K))),
        "W": fp16_round(rng.normal(0, 1.0 / 16.0, (P, K, N))),
        "bias": fp16_round(rng.normal(0, 0.01, (P, N))),
        "alpha": 0.25,
    }
