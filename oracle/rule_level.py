"""CPU oracle, rule level: one memory rule as the reference's tape sees it — an opaque block
`(embedded, level_params_flat) -> y` with the saved-buffer layout of its opaque-VJP adapter.
TEST INFRASTRUCTURE ONLY: nothing in the product path may import this module.

Restates, on top of the C++ oracle primitives:
  record_on_tape (what the forward saves)  core/src/opaque_adapters.rs:1140-1385
  {delta_rule,titans_lmm,hebbian}_opaque_backward
                                           core/src/opaque_adapters.rs:290-628
  DeltaRule / TitansLMM / HebbianRule step and step_backward
                                           core/src/delta_rule.rs:278-640, titans_lmm.rs:1314-1764
                                           (+ projection_backward :515-567), hebbian_rule.rs:91-300
  level_params_to_flat order               core/src/opaque_adapters.rs:93-113
with the identity feature map, L2 attentional bias, EMA momentum, linear memory, no conv1d and
the default (inactive) gate clamps. The memory projections multiply by the bf16-rounded copy of
W_{k,v,q}_mem (core/src/bf16.rs:54-115); their gradients go to the fp32 master.
"""
from __future__ import annotations

import numpy as np

import oracle as orc

F32 = np.float32
RULES = ("delta", "titans", "hebbian")
F32_MAX = float(np.finfo(np.float32).max)


def flat_len(d):
    """Mandatory fields of the flat parameter vector: 3 d^2 + 3 (2d + 1)."""
    return 3 * d * d + 6 * d + 3


def split_flat(flat, d):
    o, out = 0, {}
    for name, n in (("w_k_mem", d * d), ("w_v_mem", d * d), ("w_q_mem", d * d), ("w_alpha", 2 * d),
                    ("b_alpha", 1), ("w_theta", 2 * d), ("b_theta", 1), ("w_eta", 2 * d), ("b_eta", 1)):
        out[name] = np.ascontiguousarray(flat[o:o + n], dtype=F32)
        o += n
    return out


def make_flat(d, seed, b_alpha=-2.0, b_theta=-1.0, b_eta=1.5):
    r = lambda n, i, sc: orc.rand_buf(n, seed + i, sc)
    proj, gate = float(np.sqrt(2.0 / (d + d))), float(np.sqrt(1.0 / (2 * d)))
    return np.concatenate([r(d * d, 0, proj), r(d * d, 1, proj), r(d * d, 2, proj),
                           r(2 * d, 3, gate), [b_alpha], r(2 * d, 4, gate), [b_theta],
                           r(2 * d, 5, gate), [b_eta]]).astype(F32)


def _sigmoid(x):
    x = np.asarray(x, dtype=F32)
    y = (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(F32)
    return np.where(x >= 15.0, F32(1.0), np.where(x <= -15.0, F32(0.0), y)).astype(F32)


def record(rule, flat, embedded, m0=None):
    """The forward of one rule block. Returns (y, saved) with `saved` the list of buffers the
    reference's record_on_tape stores for the backward adapter, in its order."""
    assert rule in RULES
    emb = np.ascontiguousarray(embedded, dtype=F32)
    s, d = emb.shape
    p = split_flat(flat, d)
    f = lambda a: np.ascontiguousarray(a, dtype=F32)
    wk, wv, wq = (orc.bf16_round(p[n]).reshape(d, d) for n in ("w_k_mem", "w_v_mem", "w_q_mem"))
    if rule == "hebbian":
        k_mem, q_mem, kn, qn = f(emb @ wk.T), f(emb @ wq.T), None, None
    else:
        k_mem, kn = orc.l2_normalize_rows(f(emb @ wk.T))
        q_mem, qn = orc.l2_normalize_rows(f(emb @ wq.T))
    v_mem = f(emb @ wv.T)
    concat = f(np.concatenate([k_mem, v_mem], axis=1))
    alpha_pre, alpha = orc.gate(k_mem, v_mem, p["w_alpha"], float(p["b_alpha"][0]), 0)
    m0 = np.zeros(d * d, F32) if m0 is None else f(m0).ravel()
    if rule == "hebbian":
        mem = orc.hebbian_forward(k_mem, v_mem, q_mem, alpha, m0)
        meta = np.array([s, d, 0], F32)
        saved = [meta, f(flat), emb, mem["m_states"], k_mem, v_mem, q_mem, concat, alpha_pre, alpha, mem["y"]]
        return mem["y"], saved
    theta_pre, theta = orc.gate(k_mem, v_mem, p["w_theta"], float(p["b_theta"][0]), 1)
    zeros_sd, zeros_go = np.zeros((s, d), F32), np.zeros(1, F32)
    if rule == "delta":
        mem = orc.delta_forward(k_mem, v_mem, q_mem, alpha, theta, m0)
        # [seq, d, bias(L2 = 2), sign_sharpness, theta_floor, theta_ceil, fm_kind, fm_sigma,
        #  norms flag, alpha_floor, alpha_ceil, kernel_size]
        meta = np.array([s, d, 2.0, 10.0, 0.0, F32_MAX, 0.0, 1.0, 1.0, 0.0, 1.0, 0.0], F32)
        saved = [meta, f(flat), emb, mem["m_states"], k_mem, v_mem, q_mem, concat, alpha_pre, alpha,
                 theta_pre, theta, zeros_sd, zeros_go, mem["y"], kn, qn]
        return mem["y"], saved
    eta_pre, eta = orc.gate(k_mem, v_mem, p["w_eta"], float(p["b_eta"][0]), 0)
    mem = orc.titans_forward(k_mem, v_mem, q_mem, alpha, theta, eta, m0, np.zeros(d * d, F32))
    # [seq, d, bias, sign_sharpness, momentum kind (EMA = 1), theta_floor, theta_ceil, fm_kind,
    #  fm_sigma, norms flag, alpha_floor, alpha_ceil, memory_layers, expansion, activation, kernel_size]
    meta = np.array([s, d, 2.0, 10.0, 1.0, 0.0, F32_MAX, 0.0, 1.0, 1.0, 0.0, 1.0, 1.0, 4.0, 0.0, 0.0], F32)
    saved = [meta, f(flat), emb, mem["m_states"], mem["s_states"], k_mem, v_mem, q_mem, concat,
             alpha_pre, alpha, theta_pre, theta, eta_pre, eta, zeros_sd, zeros_go, mem["y"], kn, qn]
    return mem["y"], saved


def opaque_backward(rule, d_y, saved, flat_out_len=None):
    """The backward adapter: (d_embedded [s*d], d_level_params_flat [flat_out_len])."""
    meta, flat, emb = saved[0], saved[1], saved[2]
    s, d = int(meta[0]), int(meta[1])
    emb = emb.reshape(s, d)
    p = split_flat(flat, d)
    f = lambda a: np.ascontiguousarray(a, dtype=F32)
    d_y = f(d_y).reshape(s, d)
    if rule == "hebbian":
        m_states, k_mem, v_mem, q_mem, concat, alpha_pre, alpha = saved[3:10]
        b = orc.hebbian_backward(k_mem, v_mem, q_mem, alpha, m_states, d_y)
        kn = qn = None
    elif rule == "delta":
        m_states, k_mem, v_mem, q_mem, concat, alpha_pre, alpha, theta_pre, theta = saved[3:12]
        kn, qn = saved[15], saved[16]
        b = orc.delta_backward(k_mem, v_mem, q_mem, alpha, theta, m_states, d_y)
    else:
        (m_states, s_states, k_mem, v_mem, q_mem, concat, alpha_pre, alpha, theta_pre, theta,
         eta_pre, eta) = saved[3:15]
        kn, qn = saved[18], saved[19]
        b = orc.titans_backward(k_mem, v_mem, q_mem, alpha, theta, eta, m_states, s_states, d_y)
    d_k, d_v, d_q = f(b["d_k"]), f(b["d_v"]), f(b["d_q"])
    concat = concat.reshape(s, 2 * d)
    g = {n: np.zeros_like(v) for n, v in p.items()}
    gates = [("alpha", f(b["d_alpha"] * alpha * (F32(1.0) - alpha)))]
    if rule != "hebbian":
        gates.append(("theta", f(b["d_theta"] * _sigmoid(theta_pre))))
    if rule == "titans":
        gates.append(("eta", f(b["d_eta"] * eta * (F32(1.0) - eta))))
    for name, dpre in gates:
        g["w_" + name] = f(dpre @ concat)
        g["b_" + name] = np.array([dpre.sum(dtype=F32)], F32)
        d_k += np.outer(dpre, p["w_" + name][:d]).astype(F32)
        d_v += np.outer(dpre, p["w_" + name][d:]).astype(F32)
    if rule != "hebbian":
        d_k = orc.l2_normalize_rows_backward(d_k, f(k_mem).reshape(s, d), kn)
        d_q = orc.l2_normalize_rows_backward(d_q, f(q_mem).reshape(s, d), qn)
    g["w_k_mem"], g["w_v_mem"], g["w_q_mem"] = (f(x.T @ emb).ravel() for x in (d_k, d_v, d_q))
    wk, wv, wq = (orc.bf16_round(p[n]).reshape(d, d) for n in ("w_k_mem", "w_v_mem", "w_q_mem"))
    d_emb = f(d_k @ wk + d_v @ wv + d_q @ wq)
    out = np.concatenate([g[n].ravel() for n in ("w_k_mem", "w_v_mem", "w_q_mem", "w_alpha", "b_alpha",
                                                 "w_theta", "b_theta", "w_eta", "b_eta")]).astype(F32)
    n_out = out.size if flat_out_len is None else int(flat_out_len)
    padded = np.zeros(n_out, F32)
    padded[:out.size] = out
    return d_emb.ravel(), padded
