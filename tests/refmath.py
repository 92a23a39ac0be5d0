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
