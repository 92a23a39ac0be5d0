"""CPU oracle, Titans LMM with a two-layer MLP memory (deep neural memory): the inner loop of the
rule at the kernel boundary — activated gates and normalised k, v, q in; states, outputs and the
gradients of every input out. numpy, one problem at a time, a Python loop over tokens.
TEST INFRASTRUCTURE ONLY: nothing in the product path may import this module (bench.py times it
as the CPU baseline).

Restates (identity feature map, L2 attentional bias, EMA momentum, memory_layers = 2):
  MLPMemoryLayout::new                 core/src/titans_lmm.rs:65-90     packed W1[d_h,d] b1[d_h] W2[d,d_h] b2[d]
  gelu / silu / relu and derivatives   core/src/titans_lmm.rs:124-165
  mlp_forward, mlp_inner_backward,
  mlp_backward_full                    core/src/titans_lmm.rs:217-385
  TitansLMM::step_mlp (token loop)     core/src/titans_lmm.rs:771-833
  TitansLMM::step_backward_mlp
  (reverse loop, phases 1-6)           core/src/titans_lmm.rs:896-1131
  ema_step_backward                    core/src/momentum.rs:52-76
The reference's backward treats act'(pre) as a constant of the inner gradient (no second
derivative of the activation; its own finite-difference tests allow 10 %, titans_lmm.rs:2556-2585)
and passes gradients straight through the Frobenius-norm projection; both are followed here. With
ReLU the statement is the exact gradient, which is how tests/test_oracle.py pins it (float64
central differences); GELU and SiLU are pinned on the terms that do not involve act''.
The drop-in entry sums d_m_initial / d_s_initial over the batch (titans_mlp_backward.cu:557-561).
PARITY UNPINNED: the reference holds no golden vectors for this path and its Rust code cannot be
run where this was written; the pins are the finite-difference and closed-form checks named above.
"""
from __future__ import annotations

import numpy as np

ACT_GELU, ACT_SILU, ACT_RELU = 0, 1, 2


def state_size(d: int, d_hidden: int) -> int:
    return d_hidden * d + d_hidden + d * d_hidden + d


def unpack(m, d, d_hidden):
    """Views W1 [d_h,d], b1 [d_h], W2 [d,d_h], b2 [d] of one packed state."""
    o1 = d_hidden * d
    o2 = o1 + d_hidden
    o3 = o2 + d * d_hidden
    return (m[:o1].reshape(d_hidden, d), m[o1:o2], m[o2:o3].reshape(d, d_hidden), m[o3:o3 + d])


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def act(x, kind):
    if kind == ACT_GELU:
        c = x.dtype.type(0.7978845608028654)
        return x.dtype.type(0.5) * x * (1 + np.tanh(c * (x + x.dtype.type(0.044715) * x * x * x)))
    if kind == ACT_SILU:
        return x * _sigmoid(x)
    return np.maximum(x, 0)


def act_prime(x, kind):
    if kind == ACT_GELU:
        c = x.dtype.type(0.7978845608028654)
        a = x.dtype.type(0.044715)
        t = np.tanh(c * (x + a * x * x * x))
        return x.dtype.type(0.5) * (1 + t) + x.dtype.type(0.5) * x * (1 - t * t) * c * (1 + 3 * a * x * x)
    if kind == ACT_SILU:
        s = _sigmoid(x)
        return s * (1 + x * (1 - s))
    return (x > 0).astype(x.dtype)


def _mlp(m, x, d, dh, kind):
    w1, b1, w2, b2 = unpack(m, d, dh)
    pre = w1 @ x + b1
    h = act(pre, kind)
    return w2 @ h + b2, pre, h


def forward(k, v, q, alpha, theta, eta, m0, s0, d_hidden, activation=ACT_GELU, m_norm_max=0.0):
    """k, v, q [N,S,d]; gates [N,S]; m0, s0 [N,state]. Returns m_states, s_states [N,S+1,state]
    and y [N,S,d] in the dtype of k."""
    n, s, d = k.shape
    dt = k.dtype
    ss = state_size(d, d_hidden)
    ms = np.zeros((n, s + 1, ss), dt)
    sts = np.zeros((n, s + 1, ss), dt)
    y = np.zeros((n, s, d), dt)
    clamp = 0.0 < m_norm_max < 1e30
    for b in range(n):
        ms[b, 0] = m0[b]
        sts[b, 0] = s0[b]
        for t in range(s):
            m = ms[b, t]
            _, _, w2, _ = unpack(m, d, d_hidden)
            pred, pre, h = _mlp(m, k[b, t], d, d_hidden, activation)
            e = pred - v[b, t]
            gp = (w2.T @ e) * act_prime(pre, activation)
            grad = np.concatenate([np.outer(gp, k[b, t]).ravel(), gp, np.outer(e, h).ravel(), e]).astype(dt)
            sts[b, t + 1] = eta[b, t] * sts[b, t] - theta[b, t] * grad
            mn = (1 - alpha[b, t]) * m + sts[b, t + 1]
            if clamp:
                norm = np.sqrt(np.sum(mn * mn, dtype=dt))
                if norm > m_norm_max:
                    mn = mn * dt.type(m_norm_max / norm)
            ms[b, t + 1] = mn
            y[b, t] = _mlp(mn, q[b, t], d, d_hidden, activation)[0]
    return ms, sts, y


def backward(k, v, q, alpha, theta, eta, ms, sts, d_y, d_hidden, activation=ACT_GELU):
    """Reverse loop of step_backward_mlp. Returns a dict with d_k, d_v, d_q [N,S,d], d_alpha,
    d_theta, d_eta [N,S], d_m_initial, d_s_initial [N,state] (per problem; the drop-in entry adds
    them over N)."""
    n, s, d = k.shape
    dt = k.dtype
    dh = d_hidden
    ss = state_size(d, dh)
    out = dict(d_k=np.zeros((n, s, d), dt), d_v=np.zeros((n, s, d), dt), d_q=np.zeros((n, s, d), dt),
               d_alpha=np.zeros((n, s), dt), d_theta=np.zeros((n, s), dt), d_eta=np.zeros((n, s), dt),
               d_m_initial=np.zeros((n, ss), dt), d_s_initial=np.zeros((n, ss), dt))
    for b in range(n):
        dm = np.zeros(ss, dt)
        dsv = np.zeros(ss, dt)
        for t in range(s - 1, -1, -1):
            m_t, m_n, s_t = ms[b, t], ms[b, t + 1], sts[b, t]
            w1, _, w2, _ = unpack(m_t, d, dh)
            w1n, _, w2n, _ = unpack(m_n, d, dh)
            kt, vt, qt, dyt = k[b, t], v[b, t], q[b, t], d_y[b, t]
            # phase 1: readout y_t = MLP(M_{t+1}, q_t)
            _, preq, hq = _mlp(m_n, qt, d, dh, activation)
            dpq = (w2n.T @ dyt) * act_prime(preq, activation)
            dm += np.concatenate([np.outer(dpq, qt).ravel(), dpq, np.outer(dyt, hq).ravel(), dyt]).astype(dt)
            out["d_q"][b, t] = w1n.T @ dpq
            # phase 2: retention
            dsv += dm
            out["d_alpha"][b, t] = -np.dot(m_t, dm)
            dm_prev = (1 - alpha[b, t]) * dm
            # phase 3: the inner gradient of token t again
            pred, pre, h = _mlp(m_t, kt, d, dh, activation)
            e = pred - vt
            ap = act_prime(pre, activation)
            gp = (w2.T @ e) * ap
            grad = np.concatenate([np.outer(gp, kt).ravel(), gp, np.outer(e, h).ravel(), e]).astype(dt)
            # phase 4: EMA momentum
            out["d_eta"][b, t] = np.dot(s_t, dsv)
            out["d_theta"][b, t] = -np.dot(grad, dsv)
            g = -theta[b, t] * dsv
            dsv = eta[b, t] * dsv
            gw1, gb1, gw2, gb2 = unpack(g, d, dh)
            # phase 5: adjoint of the (linear in e) inner gradient, cross term, injections
            adj0 = (gw1 @ kt + gb1) * ap
            d_err = w2 @ adj0 + gw2 @ h + gb2
            inj0 = gw1.T @ gp
            inj1 = gw2.T @ e
            # phase 6: prediction path + activation path
            out["d_v"][b, t] = -d_err
            d_pre = (w2.T @ d_err + inj1) * ap
            out["d_k"][b, t] = w1.T @ d_pre + inj0
            dm_prev += np.concatenate([np.outer(d_pre, kt).ravel(), d_pre,
                                       (np.outer(d_err, h) + np.outer(e, adj0)).ravel(), d_err]).astype(dt)
            dm = dm_prev
        out["d_m_initial"][b] = dm
        out["d_s_initial"][b] = dsv
    return out


def make_problem(n, s, d, d_hidden, seed, dtype=np.float32, state_scale=0.1):
    """Seeded inputs with the reference's shapes: L2-normalised k and q rows, gates in their
    activated ranges, a small random initial MLP state, zero initial momentum."""
    rng = np.random.default_rng(seed)
    nrm = lambda a: a / np.maximum(np.linalg.norm(a, axis=-1, keepdims=True), 1e-8)
    p = dict(k=nrm(rng.standard_normal((n, s, d))), v=rng.standard_normal((n, s, d)) * 0.5,
             q=nrm(rng.standard_normal((n, s, d))), dy=rng.standard_normal((n, s, d)),
             alpha=_sigmoid(rng.standard_normal((n, s)) - 3.0),
             theta=np.log1p(np.exp(rng.standard_normal((n, s)) - 3.0)),
             eta=_sigmoid(rng.standard_normal((n, s)) + 1.5),
             m0=rng.standard_normal((n, state_size(d, d_hidden))) * state_scale,
             s0=np.zeros((n, state_size(d, d_hidden))))
    return {key: np.ascontiguousarray(val, dtype=dtype) for key, val in p.items()}


def timed_fwd_bwd(args):
    """One seeded problem forward + backward (worker of bench.py's CPU arm); returns its tokens."""
    seed, s, d, d_hidden, activation = args
    p = make_problem(1, s, d, d_hidden, seed)
    ms, sts, _ = forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], d_hidden,
                         activation)
    backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], ms, sts, p["dy"], d_hidden, activation)
    return s
