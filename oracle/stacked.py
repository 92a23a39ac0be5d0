"""CPU oracle, stacked model: n_blocks of [LN -> SWA -> W_O -> residual -> LN -> k CMS memory
levels -> softmax(alpha_mem) sum -> sigmoid gate -> residual], final LN, unembedding, cross-entropy
— forward AND backward, one sequence at a time, on top of the C++ oracle primitives (numpy for the
dense products). TEST INFRASTRUCTURE ONLY: nothing in the product path may import this module
(bench.py times it as the CPU baseline).

Restates:
  StackedMAGParams::init / BlockParams::init   core/src/stacked_model.rs:69-119,172-208
  MemoryLevelParams::init_with_depth           core/src/model.rs:462-499 (gate-bias defaults :1081-1122)
  traced_stacked_forward (+ the tape's reverse sweep over it)
                                               core/src/traced_forward.rs:1313-1499
Two level semantics (the reference's CPU and GPU paths differ here):
  mode "traced"    what traced_stacked_forward records: every level is one whole rule block on the
                   full-resolution LN_mem output with ONE d_model x d_model memory, exact per-token
                   rule, memory projections through the bf16-rounded weights (oracle/rule_level.py)
  mode "resident"  what the GPU-resident path computes (core/src/gpu_stacked_forward.rs:1656-1960,
                   gpu_forward.rs:1214-1382): level input mean-pooled by the level's chunk size,
                   fp32-master projections, L2 norm and gates at d_model resolution shared by the
                   heads, one head_dim x head_dim memory per head, level 0 exact and levels >= 1
                   frozen-M0 chunkwise, output upsampled by repetition
Parameter names follow nl_hecate_b200.stacked_mag.StackedMAG (w_qkv rows = [W_q; W_k; W_v],
w_kvq_mem rows = [W_k; W_v; W_q]_mem, w_gates rows = alpha, theta, eta).
Parity pin: float64 finite differences and the float64 forward statement in tests/test_oracle.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

import oracle as orc
from oracle import rule_level

F32 = np.float32
B_ALPHA = (3.0, 4.0, 4.5, 5.0, 5.5, 6.0)
B_THETA = (-4.6, -5.6, -6.6, -7.6, -8.6, -9.6)
B_ETA = (1.5, 2.0, 2.5, 3.0, 3.5, 4.0)


@dataclass
class Cfg:
    d_model: int = 64
    num_heads: int = 1
    n_blocks: int = 2
    k: int = 2
    chunk_sizes: tuple = (1, 8)
    seq_len: int = 32
    window: int = 32
    vocab: int = 256
    exact_levels: tuple = (0,)
    mode: str = "resident"


def init_params(cfg: Cfg, seed: int = 42):
    d, v, nb = cfg.d_model, cfg.vocab, cfg.n_blocks
    proj = math.sqrt(2.0 / (d + d))
    depth = 1.0 / math.sqrt(2.0 * nb)
    gate = math.sqrt(1.0 / (2 * d))
    emb = math.sqrt(1.0 / d)
    rng = orc.SimpleRng(seed)
    p = {"w_embed": rng.fill_uniform(v * d, emb).reshape(v, d),
         "w_unembed": rng.fill_uniform(d * v, emb).reshape(d, v),
         "ln_final_gamma": np.ones(d, F32), "ln_final_beta": np.zeros(d, F32)}
    for b in range(nb):
        pre = f"b{b}."
        bseed = seed + 10_000 + b * 10_000
        brng = orc.SimpleRng(bseed)
        p[pre + "w_qkv"] = np.concatenate([brng.fill_uniform(d * d, proj) for _ in range(3)]).reshape(3 * d, d)
        p[pre + "w_o"] = brng.fill_uniform(d * d, proj * depth).reshape(d, d)
        for n in ("ln_attn_", "ln_mem_"):
            p[pre + n + "gamma"], p[pre + n + "beta"] = np.ones(d, F32), np.zeros(d, F32)
        p[pre + "alpha_mem"] = np.zeros(cfg.k, F32)
        for l in range(cfg.k):
            q_ = pre + f"l{l}."
            lrng = orc.SimpleRng(bseed + 1000 + l * 500)
            p[q_ + "w_kvq_mem"] = np.concatenate(
                [lrng.fill_uniform(d * d, proj * depth) for _ in range(3)]).reshape(3 * d, d)
            p[q_ + "w_gates"] = np.concatenate([lrng.fill_uniform(2 * d, gate) for _ in range(3)]).reshape(3, 2 * d)
            p[q_ + "b_alpha"] = np.array([B_ALPHA[l]], F32)
            p[q_ + "b_theta"] = np.array([B_THETA[l]], F32)
            p[q_ + "b_eta"] = np.array([B_ETA[l]], F32)
    return p


def new_context(cfg: Cfg):
    """Carried memories of ONE sequence stream: [block][level] -> [heads, hd*hd] (resident) or
    [1, d*d] (traced)."""
    d = cfg.d_model
    if cfg.mode == "traced":
        return [[np.zeros((1, d * d), F32) for _ in range(cfg.k)] for _ in range(cfg.n_blocks)]
    hd = d // cfg.num_heads
    return [[np.zeros((cfg.num_heads, hd * hd), F32) for _ in range(cfg.k)] for _ in range(cfg.n_blocks)]


def _f(a):
    return np.ascontiguousarray(a, dtype=F32)


def _sigmoid(x):
    x = np.asarray(x, dtype=F32)
    y = (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(F32)
    return np.where(x >= 15.0, F32(1.0), np.where(x <= -15.0, F32(0.0), y)).astype(F32)


def _flat(p, pre):
    """Flat parameter vector of a level in the order of level_params_to_flat."""
    w, g = p[pre + "w_kvq_mem"], p[pre + "w_gates"]
    return np.concatenate([w.ravel(), g[0], p[pre + "b_alpha"], g[1], p[pre + "b_theta"], g[2],
                           p[pre + "b_eta"]]).astype(F32)


def _unflat_grads(gflat, d):
    s = rule_level.split_flat(gflat, d)
    return {"w_kvq_mem": np.concatenate([s["w_k_mem"], s["w_v_mem"], s["w_q_mem"]]).reshape(3 * d, d),
            "w_gates": np.stack([s["w_alpha"], s["w_theta"], s["w_eta"]]),
            "b_alpha": s["b_alpha"], "b_theta": s["b_theta"], "b_eta": s["b_eta"]}


# ── one CMS level, GPU-resident semantics ──────────────────────────────────
def _traj_buffers(pool, key, shape):
    """Reusable trajectory buffers of one sequence stream (the trajectories of a step live until its
    backward, so every (block, level, head) has its own pair; they are reused by the next step)."""
    if pool is None:
        return None
    if key not in pool:
        pool[key] = (np.empty(shape, F32), np.empty(shape, F32))
    return pool[key]


def _level_resident_fwd(cfg, p, pre, l, m_in, m0, pool=None):
    S, d = m_in.shape
    nh = cfg.num_heads
    hd = d // nh
    c = min(cfg.chunk_sizes[l], S)
    sf = S // c
    x = _f(m_in.reshape(sf, c, d).mean(axis=1, dtype=F32)) if c > 1 else m_in
    kvq = _f(x @ p[pre + "w_kvq_mem"].T)
    k, kn = orc.l2_normalize_rows(_f(kvq[:, :d]))
    v = _f(kvq[:, d:2 * d])
    q, qn = orc.l2_normalize_rows(_f(kvq[:, 2 * d:]))
    g = p[pre + "w_gates"]
    _, alpha = orc.gate(k, v, g[0], float(p[pre + "b_alpha"][0]), 0)
    theta_pre, theta = orc.gate(k, v, g[1], float(p[pre + "b_theta"][0]), 1)
    _, eta = orc.gate(k, v, g[2], float(p[pre + "b_eta"][0]), 0)
    exact = l in cfg.exact_levels
    chunk = min(cfg.chunk_sizes[l], sf)
    y = np.empty((sf, d), F32)
    heads, m_final = [], np.empty_like(m0)
    z = np.zeros(hd * hd, F32)
    for h in range(nh):
        sl = slice(h * hd, (h + 1) * hd)
        kh, vh, qh = _f(k[:, sl]), _f(v[:, sl]), _f(q[:, sl])
        if exact:
            f = orc.titans_forward(kh, vh, qh, alpha, theta, eta, m0[h], z,
                                   out=_traj_buffers(pool, (pre, h), (sf + 1, hd * hd)))
            m_final[h] = f["m_states"].reshape(sf + 1, -1)[-1]
        else:
            f = orc.chunkwise_forward(True, kh, vh, qh, alpha, theta, eta, m0[h], z, chunk)
            m_final[h] = f["m_chunk_states"].reshape(-1, hd * hd)[-1]
        y[:, sl] = f["y"]
        heads.append((kh, vh, qh, f))
    y_full = np.repeat(y, c, axis=0) if c > 1 else y
    cache = dict(x=x, k=k, v=v, q=q, kn=kn, qn=qn, alpha=alpha, theta=theta, theta_pre=theta_pre, eta=eta,
                 heads=heads, c=c, sf=sf, exact=exact, chunk=chunk)
    return y_full, m_final, cache


def _level_resident_bwd(cfg, p, pre, l, d_y_full, cache):
    d = cfg.d_model
    nh = cfg.num_heads
    hd = d // nh
    c, sf = cache["c"], cache["sf"]
    d_y = _f(d_y_full.reshape(sf, c, d).sum(axis=1, dtype=F32)) if c > 1 else _f(d_y_full)
    alpha, theta, eta = cache["alpha"], cache["theta"], cache["eta"]
    d_k, d_v, d_q = (np.zeros((sf, d), F32) for _ in range(3))
    d_al, d_th, d_et = (np.zeros(sf, F32) for _ in range(3))
    for h in range(nh):
        sl = slice(h * hd, (h + 1) * hd)
        kh, vh, qh, f = cache["heads"][h]
        if cache["exact"]:
            b = orc.titans_backward(kh, vh, qh, alpha, theta, eta, f["m_states"], f["s_states"], _f(d_y[:, sl]))
        else:
            b = orc.chunkwise_backward(True, kh, vh, qh, alpha, theta, eta, f["m_chunk_states"],
                                       f["s_chunk_states"], _f(d_y[:, sl]), cache["chunk"])
        d_k[:, sl], d_v[:, sl], d_q[:, sl] = b["d_k"], b["d_v"], b["d_q"]
        d_al += b["d_alpha"]; d_th += b["d_theta"]; d_et += b["d_eta"]
    g = p[pre + "w_gates"]
    concat = np.concatenate([cache["k"], cache["v"]], axis=1)
    dpre = [f32 for f32 in (_f(d_al * alpha * (F32(1.0) - alpha)), _f(d_th * _sigmoid(cache["theta_pre"])),
                            _f(d_et * eta * (F32(1.0) - eta)))]
    gw = np.stack([_f(dp @ concat) for dp in dpre])
    gb = [np.array([dp.sum(dtype=F32)], F32) for dp in dpre]
    for i, dp in enumerate(dpre):
        d_k += np.outer(dp, g[i][:d]).astype(F32)
        d_v += np.outer(dp, g[i][d:]).astype(F32)
    d_k = orc.l2_normalize_rows_backward(d_k, cache["k"], cache["kn"])
    d_q = orc.l2_normalize_rows_backward(d_q, cache["q"], cache["qn"])
    d_kvq = np.concatenate([d_k, d_v, d_q], axis=1)
    grads = {"w_kvq_mem": _f(d_kvq.T @ cache["x"]), "w_gates": gw, "b_alpha": gb[0], "b_theta": gb[1], "b_eta": gb[2]}
    d_x = _f(d_kvq @ p[pre + "w_kvq_mem"])
    d_m_in = _f(np.repeat(d_x, c, axis=0) * F32(1.0 / c)) if c > 1 else d_x
    return d_m_in, grads


# ── the model ──────────────────────────────────────────────────────────────
def forward_backward(p, ids, targets, context, cfg: Cfg, want_grads=True, pool=None):
    """One sequence. Returns (loss, grads keyed like p or None); `context` is updated in place with
    the carried memories (M of every level; S restarts at zero every call). pool: optional dict
    owned by the caller's sequence stream, holding trajectory buffers reused from step to step."""
    ids = np.asarray(ids, dtype=np.int64)
    tgt = np.asarray(targets, dtype=np.int32)
    S, d, nh = ids.shape[0], cfg.d_model, cfg.num_heads
    hd = d // nh
    w = min(cfg.window, S)
    traced = cfg.mode == "traced"
    x = _f(p["w_embed"][ids])
    blocks = []
    for b in range(cfg.n_blocks):
        pre = f"b{b}."
        h, mu1, rs1 = orc.layer_norm_forward(x, p[pre + "ln_attn_gamma"], p[pre + "ln_attn_beta"])
        qkv = _f(h @ p[pre + "w_qkv"].T)
        q, k, v = _f(qkv[:, :d]), _f(qkv[:, d:2 * d]), _f(qkv[:, 2 * d:])
        swa = orc.swa_forward(q, k, v, nh, hd, w)
        attn = swa["out"]
        attn_proj = _f(attn @ p[pre + "w_o"].T)
        res1 = _f(x + attn_proj)
        m_in, mu2, rs2 = orc.layer_norm_forward(res1, p[pre + "ln_mem_gamma"], p[pre + "ln_mem_beta"])
        wts = np.exp(p[pre + "alpha_mem"].astype(np.float64) - p[pre + "alpha_mem"].max())
        wts = (wts / wts.sum()).astype(F32)
        ys, caches = [], []
        for l in range(cfg.k):
            lp = pre + f"l{l}."
            if traced:
                y_l, saved = rule_level.record("titans", _flat(p, lp), m_in, m0=context[b][l][0])
                context[b][l][0] = saved[3].reshape(S + 1, -1)[-1]
                caches.append(saved)
            else:
                y_l, m_fin, cache = _level_resident_fwd(cfg, p, lp, l, m_in, context[b][l], pool)
                context[b][l][...] = m_fin
                caches.append(cache)
            ys.append(_f(y_l))
        y = np.zeros((S, d), F32)
        for l in range(cfg.k):
            y += wts[l] * ys[l]
        gate = _sigmoid(y)
        out = _f(x + attn_proj * gate)
        blocks.append(dict(x=x, h=h, mu1=mu1, rs1=rs1, q=q, k=k, v=v, aw=swa["attn_weights"], attn=attn,
                           attn_proj=attn_proj, res1=res1, m_in=m_in, mu2=mu2, rs2=rs2, wts=wts, ys=ys,
                           caches=caches, gate=gate))
        x = out
    xf, muf, rsf = orc.layer_norm_forward(x, p["ln_final_gamma"], p["ln_final_beta"])
    logits = _f(xf @ p["w_unembed"])
    loss_sum, count = orc.cross_entropy_sum(logits, tgt)
    loss = loss_sum / count if count > 0 else 0.0
    if not want_grads:
        return loss, None

    g = {}
    d_logits = orc.cross_entropy_backward(logits, tgt, 1.0 / max(count, 1)) if count > 0 else np.zeros_like(logits)
    g["w_unembed"] = _f(xf.T @ d_logits)
    d_xf = _f(d_logits @ p["w_unembed"].T)
    d_x, g["ln_final_gamma"], g["ln_final_beta"] = orc.layer_norm_backward(d_xf, x, p["ln_final_gamma"], muf, rsf)
    for b in range(cfg.n_blocks - 1, -1, -1):
        pre = f"b{b}."
        c = blocks[b]
        # out = x + attn_proj * sigmoid(y)
        d_attn_proj = _f(d_x * c["gate"])
        d_ycomb = _f(d_x * c["attn_proj"] * c["gate"] * (F32(1.0) - c["gate"]))
        d_res = d_x.copy()                                   # residual to the block input
        # y = sum_l softmax(alpha_mem)_l y_l
        d_w = np.array([float((d_ycomb * c["ys"][l]).sum(dtype=np.float64)) for l in range(cfg.k)])
        wts = c["wts"].astype(np.float64)
        g[pre + "alpha_mem"] = (wts * (d_w - (wts * d_w).sum())).astype(F32)
        d_m_in = np.zeros((S, d), F32)
        for l in range(cfg.k):
            lp = pre + f"l{l}."
            d_yl = _f(c["wts"][l] * d_ycomb)
            if traced:
                d_e, gflat = rule_level.opaque_backward("titans", d_yl, c["caches"][l])
                d_m_in += d_e.reshape(S, d)
                lg = _unflat_grads(gflat, d)
            else:
                d_e, lg = _level_resident_bwd(cfg, p, lp, l, d_yl, c["caches"][l])
                d_m_in += d_e
            for n, val in lg.items():
                g[lp + n] = _f(val)
        d_res1, g[pre + "ln_mem_gamma"], g[pre + "ln_mem_beta"] = orc.layer_norm_backward(
            d_m_in, c["res1"], p[pre + "ln_mem_gamma"], c["mu2"], c["rs2"])
        d_res += d_res1                                      # res1 = x + attn_proj
        d_attn_proj += d_res1
        g[pre + "w_o"] = _f(d_attn_proj.T @ c["attn"])
        d_attn = _f(d_attn_proj @ p[pre + "w_o"])
        sb = orc.swa_backward(c["q"], c["k"], c["v"], c["aw"], d_attn, nh, hd, w)
        d_qkv = np.concatenate([sb["d_q"], sb["d_k"], sb["d_v"]], axis=1)
        g[pre + "w_qkv"] = _f(d_qkv.T @ c["h"])
        d_h = _f(d_qkv @ p[pre + "w_qkv"])
        d_xa, g[pre + "ln_attn_gamma"], g[pre + "ln_attn_beta"] = orc.layer_norm_backward(
            d_h, c["x"], p[pre + "ln_attn_gamma"], c["mu1"], c["rs1"])
        d_x = _f(d_res + d_xa)
    g["w_embed"] = orc.embedding_scatter_add(d_x, ids.astype(np.int32), cfg.vocab)
    return loss, g
