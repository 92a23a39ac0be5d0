"""CPU tests that pin the oracle.

The reference ships no golden vectors; these re-create its known-answer unit
tests (cited per test) and check every analytic backward of the oracle against
central finite differences of an independent float64 statement.
"""
import numpy as np
import pytest

from refmath import fd_grad, rule_forward64


# ── known-answer pins re-created from the reference's unit tests ───────────
def test_rng_deterministic_and_range(orc):
    # core/src/tensor.rs:493-526 (determinism; fill_uniform(0.1) stays in range)
    a = orc.rand_buf(1000, 123, 0.1)
    b = orc.rand_buf(1000, 123, 0.1)
    assert np.array_equal(a, b)
    assert a.min() >= -0.1 and a.max() <= 0.1
    assert np.unique(a).size > 990


def test_rng_xorshift_known_values(orc):
    # xorshift64 (<<13, >>7, <<17) from seed 1 — computed independently in Python.
    def py_next(s):
        s ^= (s << 13) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 7
        s ^= (s << 17) & 0xFFFFFFFFFFFFFFFF
        return s
    r = orc.SimpleRng(42)
    s = 42
    for _ in range(50):
        s = py_next(s)
        assert r.next_u64() == s
    # uniform(): 2*(u as f32) - 1 scaled
    s = py_next(7)
    u = np.float32(np.float64(s) / np.float64(18446744073709551615.0))
    want = (np.float32(2.0) * u - np.float32(1.0)) * np.float32(0.5)
    assert orc.rand_buf(1, 7, 0.5)[0] == want
    toks = orc.rng_tokens(7, 256, 4)
    s = 7
    for i in range(4):
        s = py_next(s)
        assert toks[i] == s % 256


def test_sigmoid_softplus_values(orc):
    # core/src/tensor.rs:528-547
    assert abs(orc.sigmoid(0.0) - 0.5) < 1e-6
    assert orc.sigmoid(100.0) == 1.0 and orc.sigmoid(-100.0) == 0.0
    assert abs(orc.sigmoid(3.0) - 0.9526) < 1e-3
    assert abs(orc.softplus(0.0) - 0.6931) < 1e-3
    assert abs(orc.softplus(20.0) - 20.0) < 1e-2
    assert orc.softplus(-20.0) < 1e-6
    assert abs(orc.softplus(-4.6) - 0.01) < 2e-3
    # saturation thresholds are exactly +-15
    assert orc.sigmoid(15.0) == 1.0 and orc.sigmoid(14.99) < 1.0
    assert orc.softplus(15.0) == 15.0


def test_bf16_round(orc):
    # core/src/bf16.rs:183-216: powers of two exact, ~2-3 digits otherwise, zero kept.
    x = np.array([1.0, 2.0, 0.5, -4.0, 0.0, 1.234567, -3.14159], dtype=np.float32)
    r = orc.bf16_round(x)
    assert np.array_equal(r[:5], x[:5])
    assert abs(r[5] - 1.234567) < 0.01 and abs(r[6] + 3.14159) < 0.03
    # round-to-nearest-even on the tie 1 + 2^-8
    tie = np.array([1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8], dtype=np.float32)
    rt = orc.bf16_round(tie)
    assert rt[0] == 1.0 and rt[1] == np.float32(1.0 + 2.0 ** -6)
    import torch
    z = orc.rand_buf(4096, 5, 3.0)
    assert np.array_equal(orc.bf16_round(z), torch.from_numpy(z).bfloat16().float().numpy())


def test_swa_single_position_copies_v(orc):
    # core/src/swa.rs:285-299
    q = np.array([[1, 0, 0, 1]], dtype=np.float32)
    v = np.array([[0.5, 0.3, 0.1, 0.7]], dtype=np.float32)
    o = orc.swa_forward(q, q, v, 1, 4, 4)["out"]
    assert np.allclose(o, v, atol=1e-6)


def test_swa_causal_masking(orc):
    # core/src/swa.rs:301-323
    q = np.array([[1, 0], [0, 1], [1, 1]], dtype=np.float32)
    v = np.array([[1, 0], [0, 1], [0.5, 0.5]], dtype=np.float32)
    r = orc.swa_forward(q, q, v, 1, 2, 3)
    assert np.allclose(r["out"][0], [1.0, 0.0], atol=1e-5)
    assert np.isfinite(r["out"]).all()


def test_swa_window_limiting(orc):
    # core/src/swa.rs:325-344: position 3 with window 2 averages V[2], V[3]
    q = np.tile(np.array([[1.0, 0.0]], dtype=np.float32), (4, 1))
    v = np.array([[10, 0], [20, 0], [30, 0], [40, 0]], dtype=np.float32)
    o = orc.swa_forward(q, q, v, 1, 2, 2)["out"]
    assert abs(o[3, 0] - 35.0) < 1e-4


def test_swa_multi_head_weights_sum_to_one(orc):
    # core/src/swa.rs:346-378
    q = np.array([[1, 0, 0, 1], [0, 1, 1, 0]], dtype=np.float32)
    v = np.array([[0.5, 0.3, 0.1, 0.7], [0.2, 0.8, 0.4, 0.6]], dtype=np.float32)
    r = orc.swa_forward(q, q, v, 2, 2, 2)
    assert np.isfinite(r["out"]).all()
    assert np.allclose(r["attn_weights"].sum(-1), 1.0, atol=1e-5)


def test_titans_first_step_is_ema_step(orc):
    # core/src/momentum.rs:510-530: S_1 = eta*S_0 - theta*grad, grad = outer(M0 k - v, k)
    d = 4
    k, v, q = (orc.rand_buf(d, s).reshape(1, d) for s in (1, 2, 3))
    m0, s0 = orc.rand_buf(d * d, 42), orc.rand_buf(d * d, 99)
    r = orc.titans_forward(k, v, q, [0.05], [0.01], [0.9], m0, s0)
    grad = np.outer(m0.reshape(d, d) @ k[0] - v[0], k[0]).reshape(-1)
    want = np.float32(0.9) * s0 - np.float32(0.01) * grad
    assert np.allclose(r["s_states"][1], want, atol=1e-7)
    assert np.allclose(r["m_states"][1], np.float32(0.95) * m0 + r["s_states"][1], atol=1e-7)


def test_adamw_one_step_closed_form(orc):
    # core/src/adamw.rs:102-124 on one element, by hand
    w, m, v = orc.adamw_step([1.0], [0.5], [0.0], [0.0], 1e-3, 0.9, 0.999, 1e-8,
                             1 / (1 - 0.9), 1 / (1 - 0.999), 0.1)
    assert abs(m[0] - 0.05) < 1e-7 and abs(v[0] - 0.00025) < 1e-8
    # m_hat = 0.5, v_hat = 0.25 -> update = lr*(0.5/0.5 + 0.1*1)
    assert abs(w[0] - (1.0 - 1e-3 * 1.1)) < 1e-6


def test_l2_normalize_and_backward(orc):
    x = orc.rand_buf(6 * 8, 11, 1.0).reshape(6, 8)
    xn, norms = orc.l2_normalize_rows(x)
    assert np.allclose(np.linalg.norm(xn, axis=1), 1.0, atol=1e-6)
    assert np.allclose(norms, np.linalg.norm(x, axis=1), rtol=1e-6)
    go = orc.rand_buf(6 * 8, 12, 1.0).reshape(6, 8)
    gi = orc.l2_normalize_rows_backward(go, xn, norms)
    fd = fd_grad(lambda z: float((z / np.linalg.norm(z, axis=1, keepdims=True) * go).sum()), x)
    assert np.allclose(gi, fd, atol=1e-4)


# ── analytic backward vs float64 finite differences ────────────────────────
def _problem(orc, rule, s, d, seed, gates="const"):
    k = orc.rand_buf(s * d, seed, 0.5).reshape(s, d)
    v = orc.rand_buf(s * d, seed + 1, 0.5).reshape(s, d)
    q = orc.rand_buf(s * d, seed + 2, 0.5).reshape(s, d)
    dy = orc.rand_buf(s * d, seed + 3, 1.0).reshape(s, d)
    m0 = orc.rand_buf(d * d, seed + 4, 0.3)
    s0 = orc.rand_buf(d * d, seed + 5, 0.3)
    if gates == "const":
        alpha = np.full(s, 0.05, np.float32)
        theta = np.full(s, 0.01, np.float32)
        eta = np.full(s, 0.9, np.float32)
    else:
        alpha = (orc.rand_buf(s, seed + 6, 0.4) + 0.5).astype(np.float32)
        theta = (orc.rand_buf(s, seed + 7, 0.4) + 0.5).astype(np.float32)
        eta = (orc.rand_buf(s, seed + 8, 0.4) + 0.5).astype(np.float32)
    return dict(k=k, v=v, q=q, dy=dy, m0=m0, s0=s0, alpha=alpha, theta=theta, eta=eta)


def _oracle_fwd_bwd(orc, rule, p, chunk):
    if chunk:
        has_s = rule == "titans"
        f = orc.chunkwise_forward(has_s, p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"],
                                  p["m0"], p["s0"], chunk)
        b = orc.chunkwise_backward(has_s, p["k"], p["v"], p["q"], p["alpha"], p["theta"],
                                   p["eta"], f["m_chunk_states"], f["s_chunk_states"], p["dy"],
                                   chunk)
    elif rule == "titans":
        f = orc.titans_forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"],
                               p["s0"])
        b = orc.titans_backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"],
                                f["m_states"], f["s_states"], p["dy"])
    elif rule == "delta":
        f = orc.delta_forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["m0"])
        b = orc.delta_backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], f["m_states"],
                               p["dy"])
    else:
        f = orc.hebbian_forward(p["k"], p["v"], p["q"], p["alpha"], p["m0"])
        b = orc.hebbian_backward(p["k"], p["v"], p["q"], p["alpha"], f["m_states"], p["dy"])
    return f, b


@pytest.mark.parametrize("rule,chunk", [("titans", 0), ("delta", 0), ("hebbian", 0),
                                        ("titans", 3), ("delta", 3), ("titans", 4)])
def test_backward_matches_fd(orc, rule, chunk):
    s, d = 7, 4
    p = _problem(orc, rule, s, d, 100, gates="rand")
    f, b = _oracle_fwd_bwd(orc, rule, p, chunk)
    s0 = p["s0"] if rule == "titans" else None

    def loss(**over):
        a = dict(p); a.update(over)
        y, _, _ = rule_forward64(rule, a["k"], a["v"], a["q"], a["alpha"], a["theta"], a["eta"],
                                 a["m0"], a["s0"] if rule == "titans" else None, chunk)
        return float((y * p["dy"].astype(np.float64)).sum())

    y64, _, _ = rule_forward64(rule, p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"],
                               p["m0"], s0, chunk)
    assert np.allclose(f["y"], y64, atol=2e-6)
    checks = [("d_k", "k"), ("d_v", "v"), ("d_q", "q"), ("d_alpha", "alpha"),
              ("d_m_initial", "m0")]
    if rule != "hebbian":
        checks.append(("d_theta", "theta"))
    if rule == "titans":
        checks += [("d_eta", "eta"), ("d_s_initial", "s0")]
    for gname, xname in checks:
        fd = fd_grad(lambda z: loss(**{xname: z}), p[xname])
        got = b[gname].reshape(fd.shape)
        assert np.allclose(got, fd, rtol=2e-4, atol=2e-5), (rule, chunk, gname,
                                                          np.abs(got - fd).max())


def test_chunk1_equals_per_token_and_chunk4_differs(orc):
    # core/src/gpu_forward.rs:4193-4585: C=1 chunkwise == exact; C=4 differs.
    for rule in ("titans", "delta"):
        p = _problem(orc, rule, 12, 8, 300)
        fe, be = _oracle_fwd_bwd(orc, rule, p, 0)
        f1, b1 = _oracle_fwd_bwd(orc, rule, p, 1)
        f4, _ = _oracle_fwd_bwd(orc, rule, p, 4)
        assert np.allclose(fe["y"], f1["y"], atol=1e-6)
        assert np.allclose(fe["m_states"], f1["m_chunk_states"], atol=1e-6)
        for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_m_initial"):
            assert np.allclose(be[key], b1[key], atol=1e-6), key
        assert np.abs(fe["y"] - f4["y"]).max() > 1e-6


def test_error_clip_and_m_norm(orc):
    p = _problem(orc, "titans", 8, 8, 500)
    p["v"] = p["v"] * 10
    f0 = orc.titans_forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"],
                            p["s0"])
    f1 = orc.titans_forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"],
                            p["s0"], error_clip=1.0, m_norm_max=0.5)
    assert np.abs(f0["y"] - f1["y"]).max() > 1e-5
    norms = np.linalg.norm(f1["m_states"][1:], axis=1)
    assert (norms <= 0.5 + 1e-5).all()


def test_segment_seed_composition(orc):
    # backward over [0,S) == backward over [c,S) then [0,c) seeded with the first's d_M/d_S
    p = _problem(orc, "titans", 10, 4, 700, gates="rand")
    f = orc.titans_forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"],
                           p["s0"])
    full = orc.titans_backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"],
                               f["m_states"], f["s_states"], p["dy"])
    c = 6
    hi = orc.titans_backward(p["k"][c:], p["v"][c:], p["q"][c:], p["alpha"][c:], p["theta"][c:],
                             p["eta"][c:], f["m_states"][c:], f["s_states"][c:], p["dy"][c:])
    lo = orc.titans_backward(p["k"][:c], p["v"][:c], p["q"][:c], p["alpha"][:c], p["theta"][:c],
                             p["eta"][:c], f["m_states"][:c + 1], f["s_states"][:c + 1],
                             p["dy"][:c], d_m_seed=hi["d_m_initial"], d_s_seed=hi["d_s_initial"])
    assert np.allclose(np.concatenate([lo["d_k"], hi["d_k"]]), full["d_k"], atol=1e-6)
    assert np.allclose(lo["d_m_initial"], full["d_m_initial"], atol=1e-6)
    assert np.allclose(lo["d_s_initial"], full["d_s_initial"], atol=1e-6)


def test_swa_backward_matches_fd(orc):
    s, nh, hd, w = 9, 2, 4, 4
    for n_p in (0, 2):
        q, k, v, do = (orc.rand_buf(s * nh * hd, 40 + i, 0.5).reshape(s, nh * hd)
                       for i in range(4))
        f = orc.swa_forward(q, k, v, nh, hd, w, n_p)
        b = orc.swa_backward(q, k, v, f["attn_weights"], do, nh, hd, w, n_p)

        def fwd64(q_, k_, v_):
            out = np.zeros((s, nh * hd))
            for h in range(nh):
                sl = slice(h * hd, (h + 1) * hd)
                for i in range(s):
                    keys = [j for j in range(i + 1) if j < n_p or j >= max(n_p, i + 1 - w)]
                    sc = np.array([q_[i, sl] @ k_[j, sl] for j in keys]) / np.sqrt(hd)
                    pr = np.exp(sc - sc.max()); pr /= pr.sum()
                    out[i, sl] = sum(pj * v_[j, sl] for pj, j in zip(pr, keys))
            return out

        assert np.allclose(f["out"], fwd64(q, k, v), atol=2e-6)
        for name, idx in (("d_q", 0), ("d_k", 1), ("d_v", 2)):
            args = [q.astype(np.float64), k.astype(np.float64), v.astype(np.float64)]

            def loss(z, idx=idx):
                a = list(args); a[idx] = z
                return float((fwd64(*a) * do).sum())
            fd = fd_grad(loss, args[idx])
            assert np.allclose(b[name], fd, rtol=2e-4, atol=2e-5), (n_p, name)


def test_grad_norm_clip(orc):
    g = orc.rand_buf(1000, 9, 1.0)
    g2, norm, scale = orc.grad_norm_clip(g, 1.0)
    assert abs(norm - np.linalg.norm(g.astype(np.float64))) < 1e-3
    assert abs(np.linalg.norm(g2) - 1.0) < 1e-4 and scale < 1.0
    g3, _, scale3 = orc.grad_norm_clip(g, 0.0)
    assert scale3 == 1.0 and np.array_equal(g3, g)


# ── block glue (LayerNorm, cross-entropy, embedding): float64 closed forms and FD ──
def test_layer_norm_matches_float64_closed_form(orc):
    n, d = 7, 48
    x = orc.rand_buf(n * d, 901, 1.5).reshape(n, d)
    gamma = 1.0 + orc.rand_buf(d, 902, 0.3)
    beta = orc.rand_buf(d, 903, 0.2)
    out, mean, rstd = orc.layer_norm_forward(x, gamma, beta, 1e-5)
    x64 = x.astype(np.float64)
    mu = x64.mean(1, keepdims=True)
    var = ((x64 - mu) ** 2).mean(1, keepdims=True)
    ref = gamma * (x64 - mu) / np.sqrt(var + 1e-5) + beta
    assert np.abs(out - ref).max() < 5e-6
    assert np.abs(mean - mu[:, 0]).max() < 1e-6
    assert np.abs(rstd - 1 / np.sqrt(var[:, 0] + 1e-5)).max() < 1e-5


def test_layer_norm_backward_matches_finite_differences(orc):
    n, d = 3, 16
    x = orc.rand_buf(n * d, 911, 1.0).reshape(n, d).astype(np.float64)
    gamma = (1.0 + orc.rand_buf(d, 912, 0.3)).astype(np.float64)
    beta = orc.rand_buf(d, 913, 0.2).astype(np.float64)
    w = orc.rand_buf(n * d, 914, 1.0).reshape(n, d).astype(np.float64)

    def loss(x_, g_, b_):
        mu = x_.mean(1, keepdims=True)
        var = ((x_ - mu) ** 2).mean(1, keepdims=True)
        return float((w * (g_ * (x_ - mu) / np.sqrt(var + 1e-5) + b_)).sum())

    _, mean, rstd = orc.layer_norm_forward(x, gamma, beta, 1e-5)
    d_x, d_gamma, d_beta = orc.layer_norm_backward(w, x, gamma, mean, rstd)
    h = 1e-5
    for (i, j) in [(0, 0), (1, 5), (2, 15)]:
        xp, xm = x.copy(), x.copy()
        xp[i, j] += h; xm[i, j] -= h
        fd = (loss(xp, gamma, beta) - loss(xm, gamma, beta)) / (2 * h)
        assert abs(d_x[i, j] - fd) < 2e-3 * max(1.0, abs(fd))
    for j in (0, 7):
        gp, gm = gamma.copy(), gamma.copy()
        gp[j] += h; gm[j] -= h
        fd = (loss(x, gp, beta) - loss(x, gm, beta)) / (2 * h)
        assert abs(d_gamma[j] - fd) < 2e-3 * max(1.0, abs(fd))
        assert abs(d_beta[j] - w[:, j].sum()) < 1e-4


def test_cross_entropy_sum_and_gradient(orc):
    n, v = 6, 37
    logits = orc.rand_buf(n * v, 921, 3.0).reshape(n, v)
    targets = np.array([0, 36, 5, -1, 40, 12], dtype=np.int32)   # two invalid targets are skipped
    s, cnt = orc.cross_entropy_sum(logits, targets)
    l64 = logits.astype(np.float64)
    lse = np.log(np.exp(l64 - l64.max(1, keepdims=True)).sum(1)) + l64.max(1)
    valid = [i for i in range(n) if 0 <= targets[i] < v]
    ref = sum(lse[i] - l64[i, targets[i]] for i in valid)
    assert cnt == len(valid)
    assert abs(s - ref) < 1e-4
    g = orc.cross_entropy_backward(logits, targets, 1.0 / cnt)
    p = np.exp(l64 - lse[:, None])
    for i in range(n):
        if i in valid:
            e = p[i].copy(); e[targets[i]] -= 1.0
            assert np.abs(g[i] - e / cnt).max() < 1e-6
        else:
            assert np.all(g[i] == 0.0)


def test_embedding_gather_scatter_are_adjoint(orc):
    vocab, d, n = 11, 8, 9
    w = orc.rand_buf(vocab * d, 931, 1.0).reshape(vocab, d)
    ids = np.array([3, 3, 0, 10, 7, 3, 0, 1, 10], dtype=np.int32)
    out = orc.embedding_gather(w, ids)
    assert np.array_equal(out, w[ids])
    g = orc.rand_buf(n * d, 932, 1.0).reshape(n, d)
    dw = orc.embedding_scatter_add(g, ids, vocab)
    ref = np.zeros((vocab, d), np.float64)
    np.add.at(ref, ids, g.astype(np.float64))
    assert np.abs(dw - ref).max() < 1e-6


def test_oracle_reproduces_the_committed_small_vectors():
    """tests/golden/oracle_small.npz freezes the oracle's answers on seeded inputs (generated by
    tests/golden/make_golden.py; not outputs of the reference, which cannot run here). The
    oracle must reproduce them to 1e-5 relative (libm's exp/log may differ in the last bit
    between host CPUs, everything else is plain fp32 arithmetic without FMA contraction)."""
    import importlib.util
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    want = np.load(os.path.join(here, "golden", "oracle_small.npz"))
    got = mod.cases()
    assert set(got) == set(want.files)
    for key in want.files:
        a, b = np.asarray(got[key], dtype=np.float64), want[key].astype(np.float64)
        assert a.shape == b.shape and np.allclose(a, b, rtol=1e-5, atol=1e-7), key


@pytest.mark.parametrize("rule", ["delta", "titans", "hebbian"])
def test_mag_single_model_gradients_match_float64_finite_differences(orc, rule, monkeypatch):
    """The model-level oracle (oracle/mag_single.py: core/src/mag.rs mag_forward/mag_backward with
    the Delta / Titans rule wrapper) against an independent float64 statement of the loss,
    finite-differenced along random directions, one parameter tensor at a time. The memory
    projections' bf16 rounding is switched off for this test (it is a straight-through
    projection of the weights, not part of the derivative)."""
    from oracle import mag_single as M
    from refmath import mag_single_loss64
    monkeypatch.setattr(orc, "bf16_round", lambda a: np.ascontiguousarray(a, dtype=np.float32))
    d, nh, s, vocab, w = 16, 2, 12, 24, 5
    p = M.init_params(d, vocab, seed=7, rule=rule)
    for n in ("w_k_mem", "w_v_mem", "w_q_mem", "w_o"):     # make the memory branch matter
        p[n] = (p[n] * 3.0).astype(np.float32)
    p["b_alpha"][0] = -1.0
    if rule != "hebbian":
        p["b_theta"][0] = 0.3
    ids = orc.rng_tokens(11, vocab, s + 1)
    x, t = ids[:-1], ids[1:]
    loss, g = M.forward_backward(p, x, t, nh, w, rule)
    l64 = mag_single_loss64(p, x, t, nh, w, rule)
    assert abs(loss - l64) <= 1e-5 * abs(l64)
    rng = np.random.default_rng(3)
    for name in p:
        u = rng.standard_normal(p[name].shape)
        h = 1e-6
        pp = {k: v.astype(np.float64) for k, v in p.items()}
        pm = {k: v.astype(np.float64) for k, v in p.items()}
        pp[name] = pp[name] + h * u
        pm[name] = pm[name] - h * u
        fd = (mag_single_loss64(pp, x, t, nh, w, rule) - mag_single_loss64(pm, x, t, nh, w, rule)) / (2 * h)
        an = float((g[name].astype(np.float64) * u).sum())
        scale = float(np.abs(g[name]).astype(np.float64).sum()) + 1e-12
        assert abs(fd - an) <= 2e-3 * abs(fd) + 2e-5 * scale, (name, fd, an)


def _stacked_setup(orc, mode="resident", **kw):
    from oracle import stacked as ST
    cfg = ST.Cfg(d_model=16, num_heads=2, n_blocks=2, k=3, chunk_sizes=(1, 2, 8), seq_len=16, window=8,
                 vocab=32, exact_levels=(0,), mode=mode)
    for k_, v_ in kw.items():
        setattr(cfg, k_, v_)
    p = ST.init_params(cfg, seed=42)
    rng = np.random.default_rng(3)
    for n in p:                                   # make every branch matter
        base = n.split(".")[-1]
        if base.endswith("gamma"):
            p[n] = (p[n] + 0.2 * rng.standard_normal(p[n].shape)).astype(np.float32)
        elif base.endswith("beta") or base == "alpha_mem":
            p[n] = (p[n] + 0.3 * rng.standard_normal(p[n].shape)).astype(np.float32)
        elif base == "b_theta":
            p[n] = np.array([-1.0], np.float32)
        elif base == "b_alpha":
            p[n] = np.array([-2.0], np.float32)
        elif base == "w_kvq_mem":
            p[n] = (p[n] * 3.0).astype(np.float32)
    return ST, cfg, p


def test_stacked_oracle_init_follows_the_reference_streams(orc):
    """StackedMAGParams::init draw order (core/src/stacked_model.rs:69-119,172-208): one SimpleRng
    stream per scope, seeds seed / seed + 10000 (b + 1) / that + 1000 + 500 l."""
    from oracle import stacked as ST
    cfg = ST.Cfg(d_model=8, num_heads=1, n_blocks=2, k=2, chunk_sizes=(1, 2), seq_len=4, window=4, vocab=16)
    p = ST.init_params(cfg, seed=42)
    d, v = 8, 16
    top = orc.SimpleRng(42)
    assert np.array_equal(p["w_embed"].ravel(), top.fill_uniform(v * d, float(np.sqrt(1.0 / d))))
    assert np.array_equal(p["w_unembed"].ravel(), top.fill_uniform(d * v, float(np.sqrt(1.0 / d))))
    blk = orc.SimpleRng(42 + 10_000 + 10_000)                       # block 1
    proj, depth = float(np.sqrt(2.0 / (2 * d))), float(1.0 / np.sqrt(2.0 * 2))
    for i in range(3):
        assert np.array_equal(p["b1.w_qkv"][i * d:(i + 1) * d].ravel(), blk.fill_uniform(d * d, proj))
    assert np.array_equal(p["b1.w_o"].ravel(), blk.fill_uniform(d * d, proj * depth))
    lvl = orc.SimpleRng(42 + 20_000 + 1000 + 500)                   # block 1, level 1
    for i in range(3):
        assert np.array_equal(p["b1.l1.w_kvq_mem"][i * d:(i + 1) * d].ravel(), lvl.fill_uniform(d * d, proj * depth))
    for i in range(3):
        assert np.array_equal(p["b1.l1.w_gates"][i], lvl.fill_uniform(2 * d, float(np.sqrt(1.0 / (2 * d)))))
    assert p["b1.l1.b_alpha"][0] == 4.0 and p["b1.l1.b_theta"][0] == np.float32(-5.6) and p["b1.l1.b_eta"][0] == 2.0


def test_stacked_oracle_matches_float64_statement_and_finite_differences(orc):
    """oracle/stacked.py (GPU-resident level semantics, fp32) against the independent float64
    statement of the same composition: the loss over two consecutive calls (carried memories),
    and the gradient of sampled entries of EVERY parameter tensor against central differences."""
    from refmath import stacked_mag_loss64
    ST, cfg, p = _stacked_setup(orc)
    cfgd = dict(d_model=cfg.d_model, num_heads=cfg.num_heads, n_blocks=cfg.n_blocks, k=cfg.k,
                chunk_sizes=cfg.chunk_sizes, window=cfg.window, exact_levels=cfg.exact_levels)
    nh, hd = cfg.num_heads, cfg.d_model // cfg.num_heads
    ids = orc.rng_tokens(9, cfg.vocab, 2 * (cfg.seq_len + 1)).reshape(2, -1)
    ctx = ST.new_context(cfg)
    ctx64 = [[np.zeros((nh, hd * hd)) for _ in range(cfg.k)] for _ in range(cfg.n_blocks)]
    p64 = {n: a.astype(np.float64) for n, a in p.items()}
    for call in range(2):
        x, t = ids[call, :-1], ids[call, 1:]
        ctx_before = [[c.copy() for c in row] for row in ctx64]
        loss, g = ST.forward_backward(p, x, t, ctx, cfg)
        want = stacked_mag_loss64(p64, cfgd, x[None], t[None], ctx64, round_bf16=False)
        assert abs(loss - want) <= 1e-4 * abs(want), (call, loss, want)
    # finite differences at the second call (non-zero carried memory)
    rng = np.random.default_rng(0)

    def loss_at(name, idx, delta):
        q = dict(p64)
        a = q[name].copy()
        a[idx] += delta
        q[name] = a
        c = [[m.copy() for m in row] for row in ctx_before]
        return stacked_mag_loss64(q, cfgd, x[None], t[None], c, round_bf16=False)

    for name, grad in g.items():
        flat_idx = rng.choice(grad.size, size=min(3, grad.size), replace=False)
        scale = max(float(np.abs(grad).max()), 1e-8)
        for fi in flat_idx:
            idx = np.unravel_index(fi, grad.shape)
            eps = 1e-5
            fd = (loss_at(name, idx, eps) - loss_at(name, idx, -eps)) / (2 * eps)
            assert abs(grad[idx] - fd) <= 3e-3 * scale + 1e-7, (name, idx, float(grad[idx]), fd)


def test_stacked_oracle_traced_mode_equals_resident_mode_with_one_head(orc):
    """What traced_stacked_forward records (one d_model x d_model memory per level, every level an
    exact rule block on the full-resolution input, bf16-rounded projection weights) is the
    resident composition with one head, pool factor 1 and all levels exact — when the memory
    projection weights are bf16-representable, the two modes must agree."""
    ST, cfg, p = _stacked_setup(orc, num_heads=1, chunk_sizes=(1, 1, 1), exact_levels=(0, 1, 2))
    for n in p:
        if n.endswith("w_kvq_mem"):
            p[n] = orc.bf16_round(p[n].ravel()).reshape(p[n].shape)
    ids = orc.rng_tokens(11, cfg.vocab, cfg.seq_len + 1)
    x, t = ids[:-1], ids[1:]
    out = {}
    for mode in ("resident", "traced"):
        cfg.mode = mode
        ctx = ST.new_context(cfg)
        ST.forward_backward(p, x, t, ctx, cfg)               # second call sees carried memories
        out[mode] = ST.forward_backward(p, x, t, ctx, cfg)
    assert abs(out["resident"][0] - out["traced"][0]) <= 1e-6 * abs(out["traced"][0])
    for n, a in out["traced"][1].items():
        b = out["resident"][1][n]
        assert np.abs(a - b).max() <= 1e-5 * max(np.abs(a).max(), 1e-9), n


# ── MLP memory (two-layer deep memory) oracle ───────────────────────────────
def _mlp_loss(mlp, p, dh, kind):
    _, _, y = mlp.forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], dh, kind)
    return float(np.sum(y * p["dy"]))


def _mlp_fd(mlp, p, key, idx, dh, kind, eps=1e-6):
    a = p[key]
    old = a[idx]
    a[idx] = old + eps
    lp = _mlp_loss(mlp, p, dh, kind)
    a[idx] = old - eps
    lm = _mlp_loss(mlp, p, dh, kind)
    a[idx] = old
    return (lp - lm) / (2 * eps)


def test_mlp_memory_oracle_first_token_closed_form():
    """One token, zero initial momentum: S_1 = -theta * grad and M_1 = (1 - alpha) M_0 + S_1 with the
    hand-written gradient of 0.5 |MLP(k) - v|^2 (core/src/titans_lmm.rs:771-810), y = MLP(M_1, q)."""
    from oracle import mlp_memory as mlp
    d, dh = 4, 8
    p = mlp.make_problem(1, 1, d, dh, 11, np.float64)
    ms, sts, y = mlp.forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], dh,
                             mlp.ACT_SILU)
    w1, b1, w2, b2 = mlp.unpack(p["m0"][0], d, dh)
    k, v = p["k"][0, 0], p["v"][0, 0]
    pre = w1 @ k + b1
    sig = 1 / (1 + np.exp(-pre))
    h = pre * sig
    e = w2 @ h + b2 - v
    gp = (w2.T @ e) * (sig + pre * sig * (1 - sig))
    grad = np.concatenate([np.outer(gp, k).ravel(), gp, np.outer(e, h).ravel(), e])
    assert np.allclose(sts[0, 1], -p["theta"][0, 0] * grad, rtol=1e-12, atol=1e-14)
    assert np.allclose(ms[0, 1], (1 - p["alpha"][0, 0]) * p["m0"][0] + sts[0, 1], rtol=1e-12, atol=1e-14)
    w1n, b1n, w2n, b2n = mlp.unpack(ms[0, 1], d, dh)
    pq = w1n @ p["q"][0, 0] + b1n
    assert np.allclose(y[0, 0], w2n @ (pq / (1 + np.exp(-pq))) + b2n, rtol=1e-12, atol=1e-14)


def test_mlp_memory_oracle_backward_matches_float64_finite_differences_with_relu():
    """With ReLU the reference's backward (which drops the activation's second derivative) is the
    exact gradient: every output of the reverse loop against central differences of
    L = <y, d_y> in float64, momentum carried in (s0 != 0)."""
    from oracle import mlp_memory as mlp
    n, s, d, dh = 2, 5, 4, 8
    p = mlp.make_problem(n, s, d, dh, 5, np.float64, state_scale=0.5)
    p["s0"] = np.random.default_rng(6).standard_normal(p["s0"].shape) * 0.05
    kind = mlp.ACT_RELU
    ms, sts, _ = mlp.forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], dh, kind)
    g = mlp.backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], ms, sts, p["dy"], dh, kind)
    rng = np.random.default_rng(7)
    pairs = [("k", "d_k"), ("v", "d_v"), ("q", "d_q"), ("alpha", "d_alpha"), ("theta", "d_theta"),
             ("eta", "d_eta"), ("m0", "d_m_initial"), ("s0", "d_s_initial")]
    worst = 0.0
    for key, gkey in pairs:
        flat = p[key].size
        for j in rng.choice(flat, size=min(12, flat), replace=False):
            idx = np.unravel_index(j, p[key].shape)
            fd = _mlp_fd(mlp, p, key, idx, dh, kind)
            an = g[gkey][idx]
            err = abs(fd - an) / max(abs(fd), abs(an), 1e-6)
            worst = max(worst, err)
            assert err < 1e-5, (key, idx, fd, an)
    assert worst < 1e-5


@pytest.mark.parametrize("kind", [0, 1])
def test_mlp_memory_oracle_smooth_activations_exact_where_no_second_derivative_enters(kind):
    """GELU / SiLU: d_q (readout only), d_theta (first order in theta) and — with theta = 0, when the
    memory is not written — d_alpha, d_eta and the initial-state gradients do not involve act'' and
    must equal float64 central differences. (With theta > 0 the other outputs are the reference's
    approximation, not the true gradient: they are pinned by the ReLU case only.)"""
    from oracle import mlp_memory as mlp
    n, s, d, dh = 1, 4, 4, 8
    p = mlp.make_problem(n, s, d, dh, 21 + kind, np.float64, state_scale=0.5)
    p["s0"] = np.random.default_rng(8).standard_normal(p["s0"].shape) * 0.05
    rng = np.random.default_rng(9)

    def run():
        ms, sts, _ = mlp.forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], dh, kind)
        return mlp.backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], ms, sts, p["dy"], dh, kind)

    def check(pairs, tol, g):
        for key, gkey in pairs:
            for j in rng.choice(p[key].size, size=min(8, p[key].size), replace=False):
                idx = np.unravel_index(j, p[key].shape)
                fd = _mlp_fd(mlp, p, key, idx, dh, kind)
                an = g[gkey][idx]
                assert abs(fd - an) / max(abs(fd), abs(an), 1e-6) < tol, (key, idx, fd, an)

    g = run()
    last = (0, s - 1)
    for c in range(d):                      # the last token's d_q is pure readout
        fd = _mlp_fd(mlp, p, "q", last + (c,), dh, kind)
        assert abs(fd - g["d_q"][last + (c,)]) / max(abs(fd), 1e-6) < 1e-6
    fd = _mlp_fd(mlp, p, "theta", last, dh, kind)
    assert abs(fd - g["d_theta"][last]) / max(abs(fd), 1e-6) < 1e-6
    p["theta"][:] = 0.0
    g = run()
    check([("q", "d_q"), ("alpha", "d_alpha"), ("eta", "d_eta"), ("theta", "d_theta"), ("m0", "d_m_initial"),
           ("s0", "d_s_initial")], 1e-6, g)
    assert np.abs(g["d_k"]).max() == 0.0 and np.abs(g["d_v"]).max() == 0.0


def test_mlp_memory_oracle_norm_projection():
    """m_norm_max: every stored state has Frobenius norm <= the bound over the WHOLE packed state
    (core/src/titans_lmm.rs:812-821); disabled at 0 and at >= 1e30 (core/kernels/m_norm_project.cuh)."""
    from oracle import mlp_memory as mlp
    d, dh = 4, 8
    p = mlp.make_problem(2, 6, d, dh, 31, np.float32, state_scale=0.5)
    args = (p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], dh, mlp.ACT_GELU)
    ms, _, _ = mlp.forward(*args, m_norm_max=1.5)
    assert np.linalg.norm(ms[:, 1:], axis=-1).max() <= 1.5 * (1 + 1e-5)
    free, _, _ = mlp.forward(*args, m_norm_max=0.0)
    assert np.linalg.norm(free[:, 1:], axis=-1).max() > 1.5
    assert np.array_equal(free, mlp.forward(*args, m_norm_max=1e30)[0])
