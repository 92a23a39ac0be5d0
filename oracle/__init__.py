"""ctypes binding of the CPU oracle (``oracle/nlh_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: importable from ``tests/``, ``__graft_entry__.smoke``
and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``. The
product package never imports this module.

All arrays are float32 C-contiguous numpy arrays; the wrappers allocate the
outputs and return them in dicts keyed by the reference's buffer names.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, "libnlh_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile next to this file."""
    srcs = [os.path.join(_DIR, f) for f in os.listdir(_DIR) if f.endswith(".cpp")]
    stale = (not os.path.exists(_SO)) or any(
        os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", _DIR, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_sigmoid.restype = C.c_float
        _lib.orc_sigmoid.argtypes = [C.c_float]
        _lib.orc_softplus.restype = C.c_float
        _lib.orc_softplus.argtypes = [C.c_float]
        _lib.orc_grad_norm_clip.restype = C.c_float
        _lib.orc_rng_next_u64.restype = C.c_uint64
        _lib.orc_hardware_threads.restype = C.c_int
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _p(a):
    if a is None:
        return C.c_void_p(0)
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _cf(x):
    return C.c_float(float(x))


# ── RNG ────────────────────────────────────────────────────────────────────
def rand_buf(n: int, seed: int, scale: float = 0.1) -> np.ndarray:
    """``rand_buf`` of the reference's CUDA tests (core/tests/cuda_test_utils.rs:10-15)."""
    out = np.empty(n, dtype=np.float32)
    lib().orc_rng_fill_uniform(C.c_uint64(seed), _cf(scale), _p(out), C.c_int64(n))
    return out


class SimpleRng:
    """Stateful xorshift64 stream (core/src/tensor.rs:380-408)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(max(int(seed), 1))

    def fill_uniform(self, n: int, scale: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().orc_rng_stream(C.byref(self.state), _cf(scale), _p(out), C.c_int64(n))
        return out

    def next_u64(self) -> int:
        return int(lib().orc_rng_next_u64(C.byref(self.state)))


def rng_tokens(seed: int, vocab: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.int64)
    lib().orc_rng_tokens(C.c_uint64(seed), C.c_uint64(vocab), out.ctypes.data_as(C.c_void_p),
                         C.c_int64(n))
    return out


def sigmoid(x: float) -> float:
    return float(lib().orc_sigmoid(x))


def softplus(x: float) -> float:
    return float(lib().orc_softplus(x))


def bf16_round(a: np.ndarray) -> np.ndarray:
    a = _f(a)
    out = np.empty_like(a)
    lib().orc_bf16_round(_p(a), _p(out), C.c_int64(a.size))
    return out


def l2_normalize_rows(x: np.ndarray):
    x = _f(x).copy()
    n, d = x.shape
    norms = np.empty(n, dtype=np.float32)
    lib().orc_l2_normalize_rows(_p(x), _p(norms), C.c_int64(n), C.c_int64(d))
    return x, norms


def l2_normalize_rows_backward(d_out, x_norm, norms):
    d_out, x_norm, norms = _f(d_out), _f(x_norm), _f(norms)
    n, d = d_out.shape
    d_in = np.empty_like(d_out)
    lib().orc_l2_normalize_rows_backward(_p(d_out), _p(x_norm), _p(norms), _p(d_in),
                                         C.c_int64(n), C.c_int64(d))
    return d_in


def gate(k, v, w, b, which, lo=0.0, hi=0.0, has_clamp=False):
    k, v, w = _f(k), _f(v), _f(w)
    n, d = k.shape
    pre = np.empty(n, dtype=np.float32)
    out = np.empty(n, dtype=np.float32)
    lib().orc_gate(_p(k), _p(v), _p(w), _cf(b), C.c_int(which), _cf(lo), _cf(hi),
                   C.c_int(int(has_clamp)), _p(pre), _p(out), C.c_int64(n), C.c_int(d))
    return pre, out


def m_norm_clamp(m, d, batch, m_norm_max):
    m = _f(m).copy()
    lib().orc_m_norm_clamp(_p(m), C.c_int(d), C.c_int(batch), _cf(m_norm_max))
    return m


# ── memory rules: single problem ([S,d] inputs) ────────────────────────────
def delta_forward(k, v, q, alpha, theta, m0, error_clip=0.0, m_norm_max=0.0):
    k, v, q, alpha, theta, m0 = map(_f, (k, v, q, alpha, theta, m0))
    s, d = k.shape
    ms = np.empty((s + 1, d * d), dtype=np.float32)
    y = np.empty((s, d), dtype=np.float32)
    lib().orc_delta_forward(_p(k), _p(v), _p(q), _p(alpha), _p(theta), _p(m0), _p(ms), _p(y),
                            C.c_int(s), C.c_int(d), _cf(error_clip), _cf(m_norm_max))
    return {"m_states": ms, "y": y}


def delta_backward(k, v, q, alpha, theta, m_states, d_y, error_clip=0.0, d_m_seed=None):
    k, v, q, alpha, theta, m_states, d_y = map(_f, (k, v, q, alpha, theta, m_states, d_y))
    s, d = k.shape
    o = {n: np.empty((s, d), dtype=np.float32) for n in ("d_k", "d_v", "d_q")}
    o["d_alpha"] = np.empty(s, dtype=np.float32)
    o["d_theta"] = np.empty(s, dtype=np.float32)
    o["d_m_initial"] = np.empty(d * d, dtype=np.float32)
    seed = None if d_m_seed is None else _f(d_m_seed)
    lib().orc_delta_backward(_p(k), _p(v), _p(q), _p(alpha), _p(theta), _p(m_states), _p(d_y),
                             _p(seed), _p(o["d_k"]), _p(o["d_v"]), _p(o["d_q"]), _p(o["d_alpha"]),
                             _p(o["d_theta"]), _p(o["d_m_initial"]), C.c_int(s), C.c_int(d),
                             _cf(error_clip))
    return o


def titans_forward(k, v, q, alpha, theta, eta, m0, s0, error_clip=0.0, m_norm_max=0.0, out=None):
    """out: optional (m_states, s_states) float32 arrays of shape [(s+1), d*d] to write into (a
    caller that runs many steps reuses them instead of paying fresh page faults every call)."""
    k, v, q, alpha, theta, eta, m0, s0 = map(_f, (k, v, q, alpha, theta, eta, m0, s0))
    s, d = k.shape
    if out is not None:
        ms, ss = out
        assert ms.shape == (s + 1, d * d) and ss.shape == (s + 1, d * d)
    else:
        ms = np.empty((s + 1, d * d), dtype=np.float32)
        ss = np.empty((s + 1, d * d), dtype=np.float32)
    y = np.empty((s, d), dtype=np.float32)
    lib().orc_titans_forward(_p(k), _p(v), _p(q), _p(alpha), _p(theta), _p(eta), _p(m0), _p(s0),
                             _p(ms), _p(ss), _p(y), C.c_int(s), C.c_int(d), _cf(error_clip),
                             _cf(m_norm_max))
    return {"m_states": ms, "s_states": ss, "y": y}


def titans_backward(k, v, q, alpha, theta, eta, m_states, s_states, d_y, error_clip=0.0,
                    d_m_seed=None, d_s_seed=None):
    k, v, q, alpha, theta, eta, m_states, s_states, d_y = map(
        _f, (k, v, q, alpha, theta, eta, m_states, s_states, d_y))
    s, d = k.shape
    o = {n: np.empty((s, d), dtype=np.float32) for n in ("d_k", "d_v", "d_q")}
    for n in ("d_alpha", "d_theta", "d_eta"):
        o[n] = np.empty(s, dtype=np.float32)
    o["d_m_initial"] = np.empty(d * d, dtype=np.float32)
    o["d_s_initial"] = np.empty(d * d, dtype=np.float32)
    ms_ = None if d_m_seed is None else _f(d_m_seed)
    ss_ = None if d_s_seed is None else _f(d_s_seed)
    lib().orc_titans_backward(_p(k), _p(v), _p(q), _p(alpha), _p(theta), _p(eta), _p(m_states),
                              _p(s_states), _p(d_y), _p(ms_), _p(ss_), _p(o["d_k"]), _p(o["d_v"]),
                              _p(o["d_q"]), _p(o["d_alpha"]), _p(o["d_theta"]), _p(o["d_eta"]),
                              _p(o["d_m_initial"]), _p(o["d_s_initial"]), C.c_int(s), C.c_int(d),
                              _cf(error_clip))
    return o


def hebbian_forward(k, v, q, alpha, m0, m_norm_max=0.0):
    k, v, q, alpha, m0 = map(_f, (k, v, q, alpha, m0))
    s, d = k.shape
    ms = np.empty((s + 1, d * d), dtype=np.float32)
    y = np.empty((s, d), dtype=np.float32)
    lib().orc_hebbian_forward(_p(k), _p(v), _p(q), _p(alpha), _p(m0), _p(ms), _p(y), C.c_int(s),
                              C.c_int(d), _cf(m_norm_max))
    return {"m_states": ms, "y": y}


def hebbian_backward(k, v, q, alpha, m_states, d_y, d_m_seed=None):
    k, v, q, alpha, m_states, d_y = map(_f, (k, v, q, alpha, m_states, d_y))
    s, d = k.shape
    o = {n: np.empty((s, d), dtype=np.float32) for n in ("d_k", "d_v", "d_q")}
    o["d_alpha"] = np.empty(s, dtype=np.float32)
    o["d_m_initial"] = np.empty(d * d, dtype=np.float32)
    seed = None if d_m_seed is None else _f(d_m_seed)
    lib().orc_hebbian_backward(_p(k), _p(v), _p(q), _p(alpha), _p(m_states), _p(d_y), _p(seed),
                               _p(o["d_k"]), _p(o["d_v"]), _p(o["d_q"]), _p(o["d_alpha"]),
                               _p(o["d_m_initial"]), C.c_int(s), C.c_int(d))
    return o


def chunkwise_forward(has_s, k, v, q, alpha, theta, eta, m0, s0, chunk, error_clip=0.0,
                      m_norm_max=0.0):
    k, v, q, alpha, theta, m0 = map(_f, (k, v, q, alpha, theta, m0))
    s, d = k.shape
    nc = (s + chunk - 1) // chunk
    mc = np.empty((nc + 1, d * d), dtype=np.float32)
    sc = np.empty((nc + 1, d * d), dtype=np.float32) if has_s else None
    eta = _f(eta) if has_s else None
    s0 = _f(s0) if has_s else None
    y = np.empty((s, d), dtype=np.float32)
    lib().orc_chunkwise_forward(C.c_int(int(has_s)), _p(k), _p(v), _p(q), _p(alpha), _p(theta),
                                _p(eta), _p(m0), _p(s0), _p(mc), _p(sc), _p(y), C.c_int(s),
                                C.c_int(d), C.c_int(chunk), _cf(error_clip), _cf(m_norm_max))
    return {"m_chunk_states": mc, "s_chunk_states": sc, "y": y}


def chunkwise_backward(has_s, k, v, q, alpha, theta, eta, m_chunk, s_chunk, d_y, chunk,
                       error_clip=0.0, m_norm_max=0.0):
    k, v, q, alpha, theta, m_chunk, d_y = map(_f, (k, v, q, alpha, theta, m_chunk, d_y))
    s, d = k.shape
    eta = _f(eta) if has_s else None
    s_chunk = _f(s_chunk) if has_s else None
    o = {n: np.empty((s, d), dtype=np.float32) for n in ("d_k", "d_v", "d_q")}
    o["d_alpha"] = np.empty(s, dtype=np.float32)
    o["d_theta"] = np.empty(s, dtype=np.float32)
    o["d_eta"] = np.empty(s, dtype=np.float32) if has_s else None
    o["d_m_initial"] = np.empty(d * d, dtype=np.float32)
    o["d_s_initial"] = np.empty(d * d, dtype=np.float32) if has_s else None
    lib().orc_chunkwise_backward(C.c_int(int(has_s)), _p(k), _p(v), _p(q), _p(alpha), _p(theta),
                                 _p(eta), _p(m_chunk), _p(s_chunk), _p(d_y), _p(o["d_k"]),
                                 _p(o["d_v"]), _p(o["d_q"]), _p(o["d_alpha"]), _p(o["d_theta"]),
                                 _p(o["d_eta"]), _p(o["d_m_initial"]), _p(o["d_s_initial"]),
                                 C.c_int(s), C.c_int(d), C.c_int(chunk), _cf(error_clip),
                                 _cf(m_norm_max))
    return o


# ── SWA: single sequence, [S, nh*hd] ───────────────────────────────────────
def swa_forward(q, k, v, num_heads, head_dim, window, n_persistent=0):
    q, k, v = map(_f, (q, k, v))
    s = q.shape[0]
    out = np.empty_like(q)
    aw = np.empty((num_heads, s, n_persistent + window), dtype=np.float32)
    lib().orc_swa_forward(_p(q), _p(k), _p(v), _p(out), _p(aw), C.c_int(s), C.c_int(num_heads),
                          C.c_int(head_dim), C.c_int(window), C.c_int(n_persistent))
    return {"out": out, "attn_weights": aw}


def swa_backward(q, k, v, attn_weights, d_out, num_heads, head_dim, window, n_persistent=0):
    q, k, v, attn_weights, d_out = map(_f, (q, k, v, attn_weights, d_out))
    s = q.shape[0]
    o = {n: np.zeros_like(q) for n in ("d_q", "d_k", "d_v")}
    lib().orc_swa_backward(_p(q), _p(k), _p(v), _p(attn_weights), _p(d_out), _p(o["d_q"]),
                           _p(o["d_k"]), _p(o["d_v"]), C.c_int(s), C.c_int(num_heads),
                           C.c_int(head_dim), C.c_int(window), C.c_int(n_persistent))
    return o


# ── AdamW ──────────────────────────────────────────────────────────────────
def adamw_step(w, g, m, v, lr, beta1, beta2, eps, bc1_inv, bc2_inv, weight_decay):
    """In place on copies; returns (w, m, v)."""
    w, m, v = _f(w).copy(), _f(m).copy(), _f(v).copy()
    g = _f(g)
    lib().orc_adamw_step(_p(w), _p(g), _p(m), _p(v), C.c_int64(w.size), _cf(lr), _cf(beta1),
                         _cf(beta2), _cf(eps), _cf(bc1_inv), _cf(bc2_inv), _cf(weight_decay))
    return w, m, v


def grad_norm_clip(g, max_norm):
    g = _f(g).copy()
    scale = C.c_float(0)
    norm = lib().orc_grad_norm_clip(_p(g), C.c_int64(g.size), _cf(max_norm), C.byref(scale))
    return g, float(norm), float(scale.value)


def hardware_threads() -> int:
    return int(lib().orc_hardware_threads())


# ── block glue: LayerNorm, cross-entropy, embedding ────────────────────────
def _pi(a):
    assert a.dtype == np.int32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def layer_norm_forward(x, gamma, beta, eps=1e-5):
    """(out, mean, rstd) of row-wise LayerNorm over the last axis; x is [n, d]."""
    x = _f(x)
    n, d = x.shape
    out, mean, rstd = np.empty_like(x), np.empty(n, np.float32), np.empty(n, np.float32)
    lib().orc_layer_norm_forward(_p(x), _p(_f(gamma)), _p(_f(beta)), _p(out), _p(mean), _p(rstd),
                                 C.c_int(n), C.c_int(d), _cf(eps))
    return out, mean, rstd


def layer_norm_backward(d_out, x, gamma, mean, rstd):
    """(d_x, d_gamma, d_beta); the parameter gradients start from zero."""
    x, d_out = _f(x), _f(d_out)
    n, d = x.shape
    d_x, d_gamma, d_beta = np.empty_like(x), np.zeros(d, np.float32), np.zeros(d, np.float32)
    lib().orc_layer_norm_backward(_p(d_out), _p(x), _p(_f(gamma)), _p(_f(mean)), _p(_f(rstd)),
                                  _p(d_x), _p(d_gamma), _p(d_beta), C.c_int(n), C.c_int(d))
    return d_x, d_gamma, d_beta


def cross_entropy_sum(logits, targets):
    """(sum of negative log-likelihoods over valid targets, number of valid targets)."""
    logits = _f(logits)
    t = np.ascontiguousarray(targets, dtype=np.int32)
    n, v = logits.shape
    cnt = C.c_int(0)
    f = lib().orc_cross_entropy_sum
    f.restype = C.c_float
    s = f(_p(logits), _pi(t), C.c_int(n), C.c_int(v), C.byref(cnt))
    return float(s), int(cnt.value)


def cross_entropy_backward(logits, targets, inv_count):
    logits = _f(logits)
    t = np.ascontiguousarray(targets, dtype=np.int32)
    n, v = logits.shape
    d = np.empty_like(logits)
    lib().orc_cross_entropy_backward(_p(logits), _pi(t), _p(d), C.c_int(n), C.c_int(v), _cf(inv_count))
    return d


def embedding_gather(w_embed, ids):
    w = _f(w_embed)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    out = np.empty((ids.size, w.shape[1]), np.float32)
    lib().orc_embedding_gather(_p(w), _pi(ids), _p(out), C.c_int(ids.size), C.c_int(w.shape[1]))
    return out


def embedding_scatter_add(d_embedded, ids, vocab):
    g = _f(d_embedded)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    d_embed = np.zeros((vocab, g.shape[1]), np.float32)
    lib().orc_embedding_scatter_add(_p(g), _pi(ids), _p(d_embed), C.c_int(ids.size), C.c_int(g.shape[1]))
    return d_embed
