"""Shared helpers for the GPU parity tests (inputs, oracle loops, error metrics)."""
import numpy as np


def rel_err(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if want.size == 0:
        return 0.0
    assert np.isfinite(got).all(), "non-finite values in kernel output"
    denom = max(np.abs(want).max(), 1e-12)
    return float(np.abs(got - want).max() / denom)


def max_abs(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    return float(np.abs(got - want).max()) if want.size else 0.0


def make_problem(orc, n, s, d, seed, gates="const", scale=0.1, state_scale=0.1):
    """Inputs in the style of the reference's CUDA tests (core/tests/test_cuda_titans.rs:69-96):
    rand_buf(+-0.1) streams, constant gates alpha=.05 theta=.01 eta=.9; 'rand' draws gates in (0.1,0.9)."""
    r = lambda cnt, sd, sc: orc.rand_buf(cnt, sd, sc)
    p = dict(
        k=r(n * s * d, seed, scale).reshape(n, s, d),
        v=r(n * s * d, seed + 1, scale).reshape(n, s, d),
        q=r(n * s * d, seed + 2, scale).reshape(n, s, d),
        dy=r(n * s * d, seed + 3, scale).reshape(n, s, d),
        m0=r(n * d * d, seed + 4, state_scale).reshape(n, d * d),
        s0=r(n * d * d, seed + 5, state_scale).reshape(n, d * d),
    )
    if gates == "const":
        p["alpha"] = np.full((n, s), 0.05, np.float32)
        p["theta"] = np.full((n, s), 0.01, np.float32)
        p["eta"] = np.full((n, s), 0.9, np.float32)
    else:
        p["alpha"] = (r(n * s, seed + 6, 0.4) + 0.5).reshape(n, s).astype(np.float32)
        p["theta"] = (r(n * s, seed + 7, 0.4) + 0.5).reshape(n, s).astype(np.float32)
        p["eta"] = (r(n * s, seed + 8, 0.4) + 0.5).reshape(n, s).astype(np.float32)
    return p


def to_dev(p):
    import torch
    return {k: torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in p.items()}


def oracle_exact(orc, rule, p, error_clip=0.0, m_norm_max=0.0):
    """Per-problem oracle forward+backward; d_m_initial / d_s_initial summed over the batch
    (what the reference's atomicAdd produces) and also returned per problem."""
    n = p["k"].shape[0]
    fw, bw = [], []
    for b in range(n):
        if rule == "titans":
            f = orc.titans_forward(p["k"][b], p["v"][b], p["q"][b], p["alpha"][b], p["theta"][b],
                                   p["eta"][b], p["m0"][b], p["s0"][b], error_clip, m_norm_max)
            g = orc.titans_backward(p["k"][b], p["v"][b], p["q"][b], p["alpha"][b], p["theta"][b],
                                    p["eta"][b], f["m_states"], f["s_states"], p["dy"][b], error_clip)
        elif rule == "delta":
            f = orc.delta_forward(p["k"][b], p["v"][b], p["q"][b], p["alpha"][b], p["theta"][b],
                                  p["m0"][b], error_clip, m_norm_max)
            g = orc.delta_backward(p["k"][b], p["v"][b], p["q"][b], p["alpha"][b], p["theta"][b],
                                   f["m_states"], p["dy"][b], error_clip)
        else:
            f = orc.hebbian_forward(p["k"][b], p["v"][b], p["q"][b], p["alpha"][b], p["m0"][b],
                                    m_norm_max)
            g = orc.hebbian_backward(p["k"][b], p["v"][b], p["q"][b], p["alpha"][b], f["m_states"],
                                     p["dy"][b])
        fw.append(f)
        bw.append(g)
    stack = lambda lst, key: np.stack([x[key] for x in lst])
    out = {key: stack(fw, key) for key in fw[0]}
    out.update({key: stack(bw, key) for key in bw[0] if bw[0][key] is not None})
    return out


def oracle_chunkwise(orc, rule, p, chunk, error_clip=0.0, m_norm_max=0.0):
    n = p["k"].shape[0]
    has_s = rule == "titans"
    fw, bw = [], []
    for b in range(n):
        f = orc.chunkwise_forward(has_s, p["k"][b], p["v"][b], p["q"][b], p["alpha"][b],
                                  p["theta"][b], p["eta"][b], p["m0"][b], p["s0"][b], chunk,
                                  error_clip, m_norm_max)
        g = orc.chunkwise_backward(has_s, p["k"][b], p["v"][b], p["q"][b], p["alpha"][b],
                                   p["theta"][b], p["eta"][b], f["m_chunk_states"],
                                   f["s_chunk_states"], p["dy"][b], chunk, error_clip, m_norm_max)
        fw.append(f)
        bw.append(g)
    stack = lambda lst, key: np.stack([x[key] for x in lst])
    out = {key: stack(fw, key) for key in fw[0] if fw[0][key] is not None}
    out.update({key: stack(bw, key) for key in bw[0] if bw[0][key] is not None})
    return out
