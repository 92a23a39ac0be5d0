"""Independent float64 numpy statements of the recurrences, used only to
finite-difference the oracle's analytic backward passes (tests only)."""
import numpy as np


def rule_forward64(rule, k, v, q, alpha, theta, eta, m0, s0, chunk=0):
    """rule in {'titans','delta','hebbian'}; chunk>0 = frozen-M0 chunkwise.
    Returns y [S,d] (float64) and final M, S."""
    k, v, q = (np.asarray(a, dtype=np.float64) for a in (k, v, q))
    S_len, d = k.shape
    M = np.asarray(m0, dtype=np.float64).reshape(d, d).copy()
    S = None if s0 is None else np.asarray(s0, dtype=np.float64).reshape(d, d).copy()
    y = np.zeros((S_len, d))
    M0 = M.copy()
    for t in range(S_len):
        if chunk and t % chunk == 0:
            M0 = M.copy()
        a = float(alpha[t])
        if rule == "hebbian":
            M = (1 - a) * M + np.outer(v[t], k[t])
        else:
            src = M0 if chunk else M
            e = src @ k[t] - v[t]
            g = np.outer(e, k[t])
            if rule == "titans":
                S = float(eta[t]) * S - float(theta[t]) * g
                M = (1 - a) * M + S
            else:
                M = (1 - a) * M - float(theta[t]) * g
        y[t] = M @ q[t]
    return y, M, S


def fd_grad(fn, x, eps=1e-5):
    """Central finite differences of scalar fn wrt array x (float64)."""
    x = np.asarray(x, dtype=np.float64)
    g = np.zeros_like(x)
    it = np.nditer(x, flags=["multi_index"])
    while not it.finished:
        i = it.multi_index
        xp = x.copy(); xp[i] += eps
        xm = x.copy(); xm[i] -= eps
        g[i] = (fn(xp) - fn(xm)) / (2 * eps)
        it.iternext()
    return g


def swa_forward64(q, k, v, num_heads, head_dim, window):
    """Causal sliding-window attention in float64 (core/src/swa.rs:33-92): query t sees keys
    max(0, t+1-window) .. t."""
    q, k, v = (np.asarray(a, dtype=np.float64) for a in (q, k, v))
    s = q.shape[0]
    out = np.zeros_like(q)
    sc = 1.0 / np.sqrt(head_dim)
    for h in range(num_heads):
        sl = slice(h * head_dim, (h + 1) * head_dim)
        for t in range(s):
            lo = max(0, t + 1 - window)
            z = (k[lo:t + 1, sl] @ q[t, sl]) * sc
            w = np.exp(z - z.max())
            out[t, sl] = (w / w.sum()) @ v[lo:t + 1, sl]
    return out


def mag_single_loss64(p, input_ids, target_ids, num_heads, window, rule="delta"):
    """Loss of the single-block MAG model with one memory level in float64 (an independent
    statement of core/src/mag.rs:74-187 with the rule wrapper of delta_rule.rs:278-400 /
    titans_lmm.rs:1314-1530; no bf16 rounding of the memory projections)."""
    P = {k_: np.asarray(v_, dtype=np.float64) for k_, v_ in p.items()}
    ids, tgt = np.asarray(input_ids), np.asarray(target_ids)
    vocab, d = P["w_embed"].shape
    hd = d // num_heads
    emb = P["w_embed"][ids]
    attn = swa_forward64(emb @ P["w_q"].T, emb @ P["w_k"].T, emb @ P["w_v"].T, num_heads, hd, window)
    km, vm, qm = emb @ P["w_k_mem"].T, emb @ P["w_v_mem"].T, emb @ P["w_q_mem"].T
    km = km / np.maximum(np.linalg.norm(km, axis=1, keepdims=True), 1e-8)
    qm = qm / np.maximum(np.linalg.norm(qm, axis=1, keepdims=True), 1e-8)
    c = np.concatenate([km, vm], axis=1)
    sig = lambda x: 1.0 / (1.0 + np.exp(-x))
    alpha = sig(c @ P["w_alpha"] + P["b_alpha"][0])
    theta = np.log1p(np.exp(c @ P["w_theta"] + P["b_theta"][0]))
    eta = sig(c @ P["w_eta"] + P["b_eta"][0]) if rule == "titans" else None
    z = np.zeros((d, d))
    y = rule_forward64(rule, km, vm, qm, alpha, theta, eta, z, z if rule == "titans" else None)[0]
    logits = ((attn * sig(y)) @ P["w_o"].T) @ P["w_unembed"]
    m = logits.max(axis=1, keepdims=True)
    lse = np.log(np.exp(logits - m).sum(axis=1)) + m[:, 0]
    valid = [t for t in range(len(tgt)) if 0 <= tgt[t] < vocab]
    return float(np.mean([lse[t] - logits[t, tgt[t]] for t in valid]))
