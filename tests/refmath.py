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
    if rule != "hebbian":                     # the Hebbian wrapper does not normalise k, q
        km = km / np.maximum(np.linalg.norm(km, axis=1, keepdims=True), 1e-8)
        qm = qm / np.maximum(np.linalg.norm(qm, axis=1, keepdims=True), 1e-8)
    c = np.concatenate([km, vm], axis=1)
    sig = lambda x: 1.0 / (1.0 + np.exp(-x))
    alpha = sig(c @ P["w_alpha"] + P["b_alpha"][0])
    theta = np.log1p(np.exp(c @ P["w_theta"] + P["b_theta"][0])) if rule != "hebbian" else None
    eta = sig(c @ P["w_eta"] + P["b_eta"][0]) if rule == "titans" else None
    z = np.zeros((d, d))
    y = rule_forward64(rule, km, vm, qm, alpha, theta, eta, z, z if rule == "titans" else None)[0]
    logits = ((attn * sig(y)) @ P["w_o"].T) @ P["w_unembed"]
    m = logits.max(axis=1, keepdims=True)
    lse = np.log(np.exp(logits - m).sum(axis=1)) + m[:, 0]
    valid = [t for t in range(len(tgt)) if 0 <= tgt[t] < vocab]
    return float(np.mean([lse[t] - logits[t, tgt[t]] for t in valid]))


def _bf16_round64(a):
    """Round-to-nearest-even to bfloat16 precision, returned as float64."""
    a32 = np.ascontiguousarray(a, dtype=np.float32)
    u = a32.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


def _ln64(x, gamma, beta, eps=1e-5):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return gamma * (x - mu) / np.sqrt(var + eps) + beta


def stacked_mag_loss64(p, cfg, tokens, targets, context, round_bf16=True):
    """Loss of the stacked MAG model (one call = one forward over [B, S] token ids) in float64
    numpy, an independent statement of the block composition of
    core/src/gpu_stacked_forward.rs:1656-1960 as the harness runs it in its fp32 mode:
    LayerNorm -> q,k,v (rounded to bf16, as is the attention output) -> SWA -> W_o -> first
    residual -> LayerNorm -> per level: mean pool by the chunk size, k|v|q projection, L2 norm of
    k,q over d_model, three gates shared by the heads, per-head Titans memory (level 0 exact,
    levels >= 1 frozen-M0 with chunk = min(chunk size, pooled length)), repeat-upsample ->
    softmax(alpha_mem)-weighted sum -> out = x + attn_proj * sigmoid(y); final LayerNorm,
    unembedding, mean cross-entropy. `context[b][l]` ([B*H, hd*hd] float64) is the carried memory:
    read as M_0 and overwritten with the final M, like the harness does. round_bf16 = False keeps
    q, k, v and the attention output in full precision (the fp32 configuration)."""
    P = {k_: np.asarray(v_, dtype=np.float64) for k_, v_ in p.items()}
    d, nh, hd = cfg["d_model"], cfg["num_heads"], cfg["d_model"] // cfg["num_heads"]
    tok, tgt = np.asarray(tokens), np.asarray(targets)
    B, S = tok.shape
    sig = lambda z: 1.0 / (1.0 + np.exp(-z))
    x = P["w_embed"][tok]                                              # [B, S, d]
    for b in range(cfg["n_blocks"]):
        pre = f"b{b}."
        h = _ln64(x, P[pre + "ln_attn_gamma"], P[pre + "ln_attn_beta"])
        qkv = h @ P[pre + "w_qkv"].T
        if round_bf16:
            qkv = _bf16_round64(qkv)
        q, k, v = qkv[..., :d], qkv[..., d:2 * d], qkv[..., 2 * d:]
        attn = np.stack([swa_forward64(q[i], k[i], v[i], nh, hd, cfg["window"]) for i in range(B)])
        if round_bf16:
            attn = _bf16_round64(attn)
        attn_proj = attn @ P[pre + "w_o"].T
        m_in = _ln64(x + attn_proj, P[pre + "ln_mem_gamma"], P[pre + "ln_mem_beta"])
        wts = np.exp(P[pre + "alpha_mem"] - P[pre + "alpha_mem"].max())
        wts = wts / wts.sum()
        y = np.zeros_like(x)
        for l in range(cfg["k"]):
            lp = pre + f"l{l}."
            c = min(cfg["chunk_sizes"][l], S)
            sf = S // c
            xl = m_in.reshape(B, sf, c, d).mean(2) if c > 1 else m_in
            kvq = xl @ P[lp + "w_kvq_mem"].T
            km, vm, qm = kvq[..., :d], kvq[..., d:2 * d], kvq[..., 2 * d:]
            km = km / np.maximum(np.linalg.norm(km, axis=-1, keepdims=True), 1e-8)
            qm = qm / np.maximum(np.linalg.norm(qm, axis=-1, keepdims=True), 1e-8)
            pg = np.concatenate([km, vm], axis=-1) @ P[lp + "w_gates"].T       # [B, sf, 3]
            alpha = sig(pg[..., 0] + P[lp + "b_alpha"][0])
            theta = np.log1p(np.exp(pg[..., 1] + P[lp + "b_theta"][0]))
            eta = sig(pg[..., 2] + P[lp + "b_eta"][0])
            chunk = 0 if l in cfg["exact_levels"] else min(cfg["chunk_sizes"][l], sf)
            yl = np.zeros((B, sf, d))
            for i in range(B):
                for hh in range(nh):
                    sl = slice(hh * hd, (hh + 1) * hd)
                    m0 = context[b][l][i * nh + hh].reshape(hd, hd)
                    yy, m_fin, _ = rule_forward64("titans", km[i][:, sl], vm[i][:, sl], qm[i][:, sl], alpha[i],
                                                  theta[i], eta[i], m0, np.zeros((hd, hd)), chunk)
                    yl[i][:, sl] = yy
                    context[b][l][i * nh + hh] = m_fin.reshape(-1)
            y = y + wts[l] * (np.repeat(yl, c, axis=1) if c > 1 else yl)
        x = x + attn_proj * sig(y)
    x = _ln64(x, P["ln_final_gamma"], P["ln_final_beta"])
    logits = (x @ P["w_unembed"]).reshape(B * S, -1)
    m = logits.max(axis=1, keepdims=True)
    lse = np.log(np.exp(logits - m).sum(axis=1)) + m[:, 0]
    flat = tgt.reshape(-1)
    return float(np.mean(lse - logits[np.arange(B * S), flat]))
