"""CPU oracle, model level: the single-block MAG model with one memory level (k = 1) — the
reference's own CPU-runnable configuration (Delta rule + MAG, d_model 64, one head, seq 256).
TEST INFRASTRUCTURE ONLY: nothing in the product path may import this module.

Restates, stage by stage and in fp32, on top of the C++ oracle primitives:
  mag_forward                       core/src/mag.rs:74-187
  mag_backward                      core/src/mag.rs:192-392
  DeltaRule::step / step_backward   core/src/delta_rule.rs:278-640 (identity feature map, L2 bias,
                                    no conv1d, default gate clamps = none)
  TitansLMM::step / step_backward   core/src/titans_lmm.rs:1314-1764 (same wrapper, plus eta)
  HebbianRule::step / step_backward core/src/hebbian_rule.rs:91-300 (no L2 normalisation of k, q;
                                    alpha gate only)
Divergences followed as the CPU reference has them: the memory projections multiply by the
bf16-rounded copy of W_{k,v,q}_mem (core/src/bf16.rs:54-115) while gradients go to the fp32
master; the gate -> k/v gradient is included; M_0 = 0 (and S_0 = 0).
Dense products are numpy float32 matmuls (the reference's loops accumulate in another order;
differences stay at fp32 rounding level).
Parity pin: central finite differences of the loss in tests/test_oracle.py.
"""
from __future__ import annotations

import numpy as np

import oracle as orc

F32 = np.float32


def _sigmoid(x):
    """tensor.rs sigmoid_f32, saturating at +-15."""
    x = np.asarray(x, dtype=F32)
    y = (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(F32)
    return np.where(x >= 15.0, F32(1.0), np.where(x <= -15.0, F32(0.0), y)).astype(F32)


def init_params(d, vocab, seed=42, rule="delta"):
    """Seeded parameters with the reference's generator (xorshift rand_buf); scales follow the
    Xavier-style initialisation of core/src/model.rs:285-318,462-499 in spirit, not bit for bit."""
    r = lambda n, i, sc: orc.rand_buf(n, seed + i, sc)
    proj = float(np.sqrt(2.0 / (d + d)))
    p = {
        "w_embed": r(vocab * d, 0, float(np.sqrt(2.0 / (d + vocab)))).reshape(vocab, d),
        "w_unembed": r(d * vocab, 1, float(np.sqrt(2.0 / (d + vocab)))).reshape(d, vocab),
        "w_q": r(d * d, 2, proj).reshape(d, d), "w_k": r(d * d, 3, proj).reshape(d, d),
        "w_v": r(d * d, 4, proj).reshape(d, d), "w_o": r(d * d, 5, proj).reshape(d, d),
        "w_k_mem": r(d * d, 6, proj).reshape(d, d), "w_v_mem": r(d * d, 7, proj).reshape(d, d),
        "w_q_mem": r(d * d, 8, proj).reshape(d, d),
        "w_alpha": r(2 * d, 9, float(np.sqrt(1.0 / (2 * d)))), "b_alpha": np.array([-2.0], F32),
        "w_theta": r(2 * d, 10, float(np.sqrt(1.0 / (2 * d)))), "b_theta": np.array([-1.0], F32),
    }
    if rule == "titans":
        p["w_eta"] = r(2 * d, 11, float(np.sqrt(1.0 / (2 * d))))
        p["b_eta"] = np.array([1.5], F32)
    if rule == "hebbian":
        del p["w_theta"], p["b_theta"]
    return p


def forward_backward(p, input_ids, target_ids, num_heads, window, rule="delta", want_grads=True):
    """Returns (loss, grads) with grads keyed like p (None if not want_grads)."""
    ids = np.asarray(input_ids, dtype=np.int64)
    tgt = np.asarray(target_ids, dtype=np.int32)
    s = ids.shape[0]
    vocab, d = p["w_embed"].shape
    hd = d // num_heads
    f = lambda a: np.ascontiguousarray(a, dtype=F32)

    # mag.rs:97-118 embedding, q/k/v projections, SWA
    emb = f(p["w_embed"][ids])
    q, k, v = f(emb @ p["w_q"].T), f(emb @ p["w_k"].T), f(emb @ p["w_v"].T)
    swa = orc.swa_forward(q, k, v, num_heads, hd, window)
    attn_out = swa["out"]

    # memory branch: delta_rule.rs:286-304 / titans_lmm.rs:1333-1362
    wk16, wv16, wq16 = (orc.bf16_round(p[n]) for n in ("w_k_mem", "w_v_mem", "w_q_mem"))
    hebbian = rule == "hebbian"
    if hebbian:                                   # hebbian_rule.rs:111-118: raw projections
        k_mem, q_mem, kn, qn = f(emb @ wk16.T), f(emb @ wq16.T), None, None
    else:
        k_mem, kn = orc.l2_normalize_rows(f(emb @ wk16.T))
        q_mem, qn = orc.l2_normalize_rows(f(emb @ wq16.T))
    v_mem = f(emb @ wv16.T)
    alpha_pre, alpha = orc.gate(k_mem, v_mem, p["w_alpha"], float(p["b_alpha"][0]), 0)
    if not hebbian:
        theta_pre, theta = orc.gate(k_mem, v_mem, p["w_theta"], float(p["b_theta"][0]), 1)
    m0 = np.zeros(d * d, F32)
    if hebbian:
        mem = orc.hebbian_forward(k_mem, v_mem, q_mem, alpha, m0)
    elif rule == "titans":
        eta_pre, eta = orc.gate(k_mem, v_mem, p["w_eta"], float(p["b_eta"][0]), 0)
        mem = orc.titans_forward(k_mem, v_mem, q_mem, alpha, theta, eta, m0, m0)
    else:
        mem = orc.delta_forward(k_mem, v_mem, q_mem, alpha, theta, m0)
    y = mem["y"]

    # mag.rs:158-181 gating, output projection, unembedding, loss
    gate = _sigmoid(y)
    gated = f(attn_out * gate)
    projected = f(gated @ p["w_o"].T)
    logits = f(projected @ p["w_unembed"])
    loss_sum, count = orc.cross_entropy_sum(logits, tgt)
    loss = loss_sum / count if count > 0 else 0.0
    if not want_grads:
        return loss, None

    # mag.rs:215-262
    g = {}
    d_logits = orc.cross_entropy_backward(logits, tgt, 1.0 / max(count, 1)) if count > 0 else np.zeros_like(logits)
    d_projected = f(d_logits @ p["w_unembed"].T)
    g["w_unembed"] = f(projected.T @ d_logits)
    d_gated = f(d_projected @ p["w_o"])
    g["w_o"] = f(d_projected.T @ gated)
    d_attn = f(d_gated * gate)
    d_y = f(d_gated * attn_out * gate * (F32(1.0) - gate))

    # memory backward: delta_rule.rs:420-640 / titans_lmm.rs:1535-1764
    if hebbian:
        b = orc.hebbian_backward(k_mem, v_mem, q_mem, alpha, mem["m_states"], d_y)
    elif rule == "titans":
        b = orc.titans_backward(k_mem, v_mem, q_mem, alpha, theta, eta, mem["m_states"], mem["s_states"], d_y)
    else:
        b = orc.delta_backward(k_mem, v_mem, q_mem, alpha, theta, mem["m_states"], d_y)
    d_k, d_v, d_q = f(b["d_k"]), f(b["d_v"]), f(b["d_q"])
    concat = np.concatenate([k_mem, v_mem], axis=1)
    d_alpha_pre = f(b["d_alpha"] * alpha * (F32(1.0) - alpha))
    gates = [("alpha", d_alpha_pre)]
    if not hebbian:
        gates.append(("theta", f(b["d_theta"] * _sigmoid(theta_pre))))   # softplus' = sigmoid; clamp mask = 1
    if rule == "titans":
        gates.append(("eta", f(b["d_eta"] * eta * (F32(1.0) - eta))))
    for name, dpre in gates:
        g["w_" + name] = f(dpre @ concat)
        g["b_" + name] = np.array([dpre.sum(dtype=F32)], F32)
        d_k += np.outer(dpre, p["w_" + name][:d]).astype(F32)       # gate -> k/v gradient
        d_v += np.outer(dpre, p["w_" + name][d:]).astype(F32)
    d_k_raw = d_k if hebbian else orc.l2_normalize_rows_backward(d_k, k_mem, kn)
    d_q_raw = d_q if hebbian else orc.l2_normalize_rows_backward(d_q, q_mem, qn)
    g["w_k_mem"], g["w_v_mem"], g["w_q_mem"] = f(d_k_raw.T @ emb), f(d_v.T @ emb), f(d_q_raw.T @ emb)
    d_emb = f(d_k_raw @ wk16 + d_v @ wv16 + d_q_raw @ wq16)

    # attention backward: mag.rs:341-372
    sb = orc.swa_backward(q, k, v, swa["attn_weights"], d_attn, num_heads, hd, window)
    d_emb += f(sb["d_q"] @ p["w_q"] + sb["d_k"] @ p["w_k"] + sb["d_v"] @ p["w_v"])
    g["w_q"], g["w_k"], g["w_v"] = f(sb["d_q"].T @ emb), f(sb["d_k"].T @ emb), f(sb["d_v"].T @ emb)
    g["w_embed"] = orc.embedding_scatter_add(d_emb, ids.astype(np.int32), vocab)
    return loss, g
