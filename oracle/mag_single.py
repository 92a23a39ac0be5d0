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
from oracle import rule_level

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

    # memory branch: the rule block as the tape records it (oracle/rule_level.py restates
    # delta_rule.rs:286-304 / titans_lmm.rs:1333-1362 / hebbian_rule.rs:111-118)
    z2, z1 = np.zeros(2 * d, F32), np.zeros(1, F32)
    flat = np.concatenate([p["w_k_mem"].ravel(), p["w_v_mem"].ravel(), p["w_q_mem"].ravel(),
                           p["w_alpha"], p["b_alpha"], p.get("w_theta", z2), p.get("b_theta", z1),
                           p.get("w_eta", z2), p.get("b_eta", z1)]).astype(F32)
    y, saved = rule_level.record(rule, flat, emb)

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

    # memory backward: delta_rule.rs:420-640 / titans_lmm.rs:1535-1764 through the adapter
    d_emb, gflat = rule_level.opaque_backward(rule, d_y, saved)
    d_emb = f(d_emb.reshape(s, d))
    for name, val in rule_level.split_flat(gflat, d).items():
        if name in p:
            g[name] = val.reshape(p[name].shape)

    # attention backward: mag.rs:341-372
    sb = orc.swa_backward(q, k, v, swa["attn_weights"], d_attn, num_heads, hd, window)
    d_emb += f(sb["d_q"] @ p["w_q"] + sb["d_k"] @ p["w_k"] + sb["d_v"] @ p["w_v"])
    g["w_q"], g["w_k"], g["w_v"] = f(sb["d_q"].T @ emb), f(sb["d_k"].T @ emb), f(sb["d_v"].T @ emb)
    g["w_embed"] = orc.embedding_scatter_add(d_emb, ids.astype(np.int32), vocab)
    return loss, g
