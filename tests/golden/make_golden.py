"""Writes tests/golden/oracle_small.npz: small known-answer vectors produced by the CPU oracle.

The reference is a Rust workspace that cannot be built where this repository is developed and
ships no golden vectors of its own, so these fixtures are NOT outputs of the reference: they
freeze the oracle's answers on seeded inputs (the reference's own rand_buf generator) so that a
later change to the oracle — or, on a machine with the reference's toolchain, a difference from
the reference — shows up as a failing comparison. Regenerate with

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as orc  # noqa: E402


def cases():
    out = {}
    d, s = 8, 6
    r = lambda n, seed, sc=0.1: orc.rand_buf(n, seed, sc)
    k, v, q, dy = (r(s * d, 100 + i).reshape(s, d) for i in range(4))
    m0, s0 = r(d * d, 104), r(d * d, 105)
    al, th, et = np.full(s, 0.05, np.float32), np.full(s, 0.01, np.float32), np.full(s, 0.9, np.float32)
    f = orc.titans_forward(k, v, q, al, th, et, m0, s0)
    b = orc.titans_backward(k, v, q, al, th, et, f["m_states"], f["s_states"], dy)
    out.update({"titans_y": f["y"], "titans_m_final": f["m_states"][-1], "titans_s_final": f["s_states"][-1]})
    out.update({"titans_" + key: np.asarray(val) for key, val in b.items()})
    f = orc.delta_forward(k, v, q, al, th, m0)
    b = orc.delta_backward(k, v, q, al, th, f["m_states"], dy)
    out.update({"delta_y": f["y"], "delta_m_final": f["m_states"][-1]})
    out.update({"delta_" + key: np.asarray(val) for key, val in b.items()})
    f = orc.hebbian_forward(k, v, q, al, m0)
    b = orc.hebbian_backward(k, v, q, al, f["m_states"], dy)
    out.update({"hebbian_y": f["y"]})
    out.update({"hebbian_" + key: np.asarray(val) for key, val in b.items()})
    s2, c = 8, 4
    k2, v2, q2, dy2 = (r(s2 * d, 200 + i).reshape(s2, d) for i in range(4))
    al2, th2, et2 = (np.full(s2, x, np.float32) for x in (0.05, 0.01, 0.9))
    f = orc.chunkwise_forward(True, k2, v2, q2, al2, th2, et2, m0, s0, c)
    b = orc.chunkwise_backward(True, k2, v2, q2, al2, th2, et2, f["m_chunk_states"], f["s_chunk_states"], dy2, c)
    out.update({"chunk_y": f["y"], "chunk_m_chunk": f["m_chunk_states"]})
    out.update({"chunk_" + key: np.asarray(val) for key, val in b.items()})
    sq, nh, hd, w = 12, 2, 4, 5
    qa, ka, va, do = (r(sq * nh * hd, 300 + i, 0.5).reshape(sq, nh * hd) for i in range(4))
    f = orc.swa_forward(qa, ka, va, nh, hd, w)
    b = orc.swa_backward(qa, ka, va, f["attn_weights"], do, nh, hd, w)
    out.update({"swa_out": f["out"], "swa_attn_weights": f["attn_weights"]})
    out.update({"swa_" + key: np.asarray(val) for key, val in b.items()})
    n = 37
    w_, g_, m_, v_ = r(n, 400, 1.0), r(n, 401, 0.1), r(n, 402, 0.01), np.abs(r(n, 403, 0.001))
    w1, m1, v1 = orc.adamw_step(w_, g_, m_, v_, 3e-4, 0.9, 0.999, 1e-8, 10.0, 1000.0, 0.1)
    out.update({"adamw_w": w1, "adamw_m": m1, "adamw_v": v1})
    x = r(5 * 12, 500, 1.5).reshape(5, 12)
    gamma, beta = 1.0 + r(12, 501, 0.3), r(12, 502, 0.2)
    o, mean, rstd = orc.layer_norm_forward(x, gamma, beta, 1e-5)
    dx, dg, db = orc.layer_norm_backward(r(60, 503, 1.0).reshape(5, 12), x, gamma, mean, rstd)
    out.update({"ln_out": o, "ln_dx": dx, "ln_dgamma": dg, "ln_dbeta": db})
    logits = r(4 * 9, 600, 3.0).reshape(4, 9)
    tg = np.array([0, 8, 3, 11], dtype=np.int32)
    ssum, cnt = orc.cross_entropy_sum(logits, tg)
    out.update({"ce_sum": np.array([ssum], np.float32), "ce_grad": orc.cross_entropy_backward(logits, tg, 1.0 / cnt)})
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_small.npz")
    np.savez_compressed(path, **cases())
    print(path, os.path.getsize(path), "bytes")
