"""GPU parity: memory-rule kernels (through the C ABI) vs the CPU oracle.

Tolerances: forward max-abs 1e-5 and backward max-abs 1e-4 on +-0.1 inputs are
the reference's own (core/tests/test_cuda_titans.rs:1-4,94-96); relative error
<= 1e-4 (max-abs error over max-abs reference) is the fp32 bar of the hot path.
Head dims 32 and 64 without clip/projection run the register-resident kernels,
everything else the generic-d kernels; both are covered.
"""
import numpy as np
import pytest

from helpers import make_problem, max_abs, oracle_chunkwise, oracle_exact, rel_err, to_dev

pytestmark = pytest.mark.gpu

REL = 1e-4


@pytest.fixture(scope="module")
def D():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch
    return dispatch


def _np(t):
    return t.detach().cpu().numpy()


def _check_bwd(got, want, keys, tol_abs=1e-4):
    for key in keys:
        g = _np(got[key])
        w = want[key]
        if key in ("d_m_initial", "d_s_initial") and g.ndim == 1:
            w = w.sum(0)   # the drop-in entries sum the initial-state grads over the batch
        assert rel_err(g, w) <= REL, (key, rel_err(g, w))
        assert max_abs(g, w) < tol_abs, (key, max_abs(g, w))


@pytest.mark.parametrize("d,s,n", [(8, 12, 1), (16, 16, 3), (4, 1, 2), (32, 8, 2), (32, 21, 1),
                                   (64, 16, 2), (64, 37, 3), (64, 1, 1), (128, 8, 1)])
@pytest.mark.parametrize("gates", ["const", "rand"])
def test_titans_exact(D, orc, d, s, n, gates):
    p = make_problem(orc, n, s, d, 100 + d + s, gates)
    w = oracle_exact(orc, "titans", p)
    t = to_dev(p)
    ms, ss, y = D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                                    t["m0"], t["s0"])
    assert max_abs(_np(y), w["y"]) < 1e-5 and rel_err(_np(y), w["y"]) <= REL
    assert rel_err(_np(ms), w["m_states"]) <= REL and rel_err(_np(ss), w["s_states"]) <= REL
    g = D.titans_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], ms, ss,
                             t["dy"])
    _check_bwd(g, w, ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta", "d_m_initial",
                      "d_s_initial"])


@pytest.mark.parametrize("d,s,n", [(8, 12, 2), (16, 8, 1), (32, 19, 2), (64, 16, 2), (64, 45, 1)])
@pytest.mark.parametrize("dgd", [False, True])
def test_delta_and_dgd_exact(D, orc, d, s, n, dgd):
    if dgd:
        n = 1   # dgd_backward_f32_cuda has no batch argument (core/src/cuda_ffi.rs:309)
    p = make_problem(orc, n, s, d, 300 + d + s, "rand")
    w = oracle_exact(orc, "delta", p)
    t = to_dev(p)
    ms, y = D.delta_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["m0"], dgd=dgd)
    assert max_abs(_np(y), w["y"]) < 1e-5 and rel_err(_np(ms), w["m_states"]) <= REL
    g = D.delta_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], ms, t["dy"], dgd=dgd)
    _check_bwd(g, w, ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_m_initial"])


@pytest.mark.parametrize("d,s", [(8, 12), (32, 9), (64, 16), (64, 33)])
def test_hebbian_exact(D, orc, d, s):
    p = make_problem(orc, 1, s, d, 500 + d + s, "rand")
    w = oracle_exact(orc, "hebbian", p)
    t = to_dev(p)
    ms, y = D.hebbian_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["m0"])
    assert max_abs(_np(y), w["y"]) < 1e-5 and rel_err(_np(ms), w["m_states"]) <= REL
    g = D.hebbian_backward_dd(t["k"], t["v"], t["q"], t["alpha"], ms, t["dy"])
    _check_bwd(g, w, ["d_k", "d_v", "d_q", "d_alpha", "d_m_initial"])


def test_hebbian_forward_batched(D, orc):
    p = make_problem(orc, 3, 10, 64, 540, "rand")
    w = oracle_exact(orc, "hebbian", p)
    t = to_dev(p)
    ms, y = D.hebbian_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["m0"])
    assert rel_err(_np(y), w["y"]) <= REL and rel_err(_np(ms), w["m_states"]) <= REL


@pytest.mark.parametrize("d", [16, 64])
def test_titans_clip_and_projection(D, orc, d):
    # error_clip=1, m_norm_max=5 with large v so that both trigger
    # (core/tests/test_cuda_titans.rs:420-467)
    p = make_problem(orc, 2, 12, d, 700 + d, "const", scale=1.0, state_scale=1.0)
    w = oracle_exact(orc, "titans", p, error_clip=1.0, m_norm_max=5.0)
    w0 = oracle_exact(orc, "titans", p)
    assert np.abs(w["y"] - w0["y"]).max() > 1e-3   # the options changed the result
    t = to_dev(p)
    ms, ss, y = D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                                    t["m0"], t["s0"], error_clip=1.0, m_norm_max=5.0)
    assert rel_err(_np(y), w["y"]) <= REL and rel_err(_np(ms), w["m_states"]) <= REL
    g = D.titans_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], ms, ss,
                             t["dy"], error_clip=1.0)
    for key in ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"]:
        assert rel_err(_np(g[key]), w[key]) <= REL, key


@pytest.mark.parametrize("rule", ["titans", "delta"])
@pytest.mark.parametrize("d,s,chunk,n", [(8, 12, 4, 2), (16, 10, 3, 1), (32, 24, 8, 2),
                                         (64, 64, 64, 2), (64, 50, 16, 2), (64, 9, 1, 1),
                                         (64, 130, 64, 1), (64, 8, 512, 1), (64, 100, 24, 3),
                                         (64, 37, 33, 2), (64, 200, 48, 2), (64, 17, 17, 1)])
def test_chunkwise(D, orc, rule, d, s, chunk, n):
    p = make_problem(orc, n, s, d, 900 + d + s + chunk, "rand")
    w = oracle_chunkwise(orc, rule, p, chunk)
    t = to_dev(p)
    if rule == "titans":
        mc, sc, y = D.titans_chunkwise_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"],
                                                  t["eta"], t["m0"], t["s0"], chunk)
        assert rel_err(_np(sc), w["s_chunk_states"]) <= REL
        g = D.titans_chunkwise_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"],
                                           t["eta"], mc, sc, t["dy"], chunk)
        keys = ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta", "d_m_initial", "d_s_initial"]
    else:
        mc, y = D.delta_chunkwise_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"],
                                             t["m0"], chunk)
        g = D.delta_chunkwise_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], mc,
                                          t["dy"], chunk)
        keys = ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_m_initial"]
    assert rel_err(_np(y), w["y"]) <= REL
    assert rel_err(_np(mc), w["m_chunk_states"]) <= REL
    _check_bwd(g, w, keys, tol_abs=1e-3)


def test_chunk_matrix_form_matches_per_token_kernels(D, orc):
    """Chunk sizes 16..64 at head_dim 64 run the chunk-parallel matrix form (contractions over the
    chunk instead of a token loop); option NLH_OPT_CHUNK_MATRIX = 0 selects the per-token kernels.
    Both must agree with each other (they are compared with the oracle in test_chunkwise)."""
    p = make_problem(orc, 3, 150, 64, 4100, "rand")
    t = to_dev(p)
    res = []
    for on in (1, 0):
        D.call("nlh_set_option", option=2, value=on)
        try:
            mc, sc, y = D.titans_chunkwise_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"],
                                                      t["eta"], t["m0"], t["s0"], 40)
            g = D.titans_chunkwise_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"],
                                               t["eta"], mc, sc, t["dy"], 40)
        finally:
            D.call("nlh_set_option", option=2, value=1)
        res.append(dict(g, y=y, mc=mc, sc=sc))
    for key in res[0]:
        assert rel_err(_np(res[0][key]), _np(res[1][key])) <= REL, key


def test_chunk1_matches_per_token_kernel(D, orc):
    # core/src/gpu_forward.rs:4193-4300: C=1 chunkwise == per-token kernel (<1e-5)
    p = make_problem(orc, 2, 16, 64, 1200, "const")
    t = to_dev(p)
    ms, ss, y = D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                                    t["m0"], t["s0"])
    mc, sc, yc = D.titans_chunkwise_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"],
                                               t["eta"], t["m0"], t["s0"], 1)
    assert max_abs(_np(y), _np(yc)) < 1e-5
    assert max_abs(_np(ms), _np(mc)) < 1e-5 and max_abs(_np(ss), _np(sc)) < 1e-5


def test_chunkwise_with_clip_uses_generic_path(D, orc):
    p = make_problem(orc, 2, 20, 64, 1300, "rand", scale=1.0, state_scale=0.5)
    w = oracle_chunkwise(orc, "titans", p, 8, error_clip=1.0, m_norm_max=4.0)
    t = to_dev(p)
    mc, sc, y = D.titans_chunkwise_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"],
                                              t["eta"], t["m0"], t["s0"], 8, 1.0, 4.0)
    assert rel_err(_np(y), w["y"]) <= REL
    g = D.titans_chunkwise_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                                       mc, sc, t["dy"], 8, 1.0, 4.0)
    for key in ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"]:
        assert rel_err(_np(g[key]), w[key]) <= REL, key


@pytest.mark.parametrize("rule", ["titans", "delta", "hebbian"])
@pytest.mark.parametrize("d,s,interval", [(16, 12, 4), (64, 24, 8), (64, 19, 4), (32, 7, 16)])
def test_checkpoint_forward_and_segment_backward(D, orc, rule, d, s, interval):
    """*_forward_ckpt stores state 0, every `interval` tokens and the final state; the
    backward is replayed segment by segment with seeds (core/tests/test_gradient_checkpoint.rs,
    replay logic of core/src/gpu_backward.rs:1770-1965)."""
    import torch
    p = make_problem(orc, 1, s, d, 1500 + d + s, "rand")
    w = oracle_exact(orc, rule, p)
    t = to_dev(p)
    nck = D.checkpoint_count(s, interval)
    dev = t["k"].device
    f32 = lambda *sh: torch.empty(*sh, dtype=torch.float32, device=dev)
    mck, sck, y = f32(nck, d * d), f32(nck, d * d), f32(s, d)
    k1, v1, q1 = t["k"][0], t["v"][0], t["q"][0]
    a1, th1, e1 = t["alpha"][0], t["theta"][0], t["eta"][0]
    if rule == "titans":
        D.call("titans_forward_ckpt_f32_cuda", k_mem=k1, v_mem=v1, q_mem=q1, alpha=a1, theta=th1,
               eta=e1, m_initial=t["m0"], s_initial=t["s0"], m_states=mck, s_states=sck, y=y,
               seq_len=s, d=d, checkpoint_interval=interval, error_clip=0.0, m_norm_max=0.0)
    elif rule == "delta":
        D.call("delta_forward_ckpt_f32_cuda", k_mem=k1, v_mem=v1, q_mem=q1, alpha=a1, theta=th1,
               m_initial=t["m0"], m_states=mck, y=y, seq_len=s, d=d,
               checkpoint_interval=interval, error_clip=0.0, m_norm_max=0.0)
    else:
        D.call("hebbian_forward_ckpt_f32_cuda", k_mem=k1, v_mem=v1, q_mem=q1, alpha=a1,
               m_initial=t["m0"], m_states=mck, y=y, seq_len=s, d=d, checkpoint_interval=interval)
    assert rel_err(_np(y), w["y"][0]) <= REL
    bounds = [0] + [tt + 1 for tt in range(s) if (tt + 1) % interval == 0 or tt + 1 == s]
    assert len(bounds) == nck
    assert rel_err(_np(mck), w["m_states"][0][bounds]) <= REL
    if rule == "titans":
        assert rel_err(_np(sck), w["s_states"][0][bounds]) <= REL

    # segment replay: re-run the full-trajectory forward on each segment from its checkpoint
    dk, dv, dq = (torch.zeros(1, s, d, device=dev) for _ in range(3))
    da, dth, de = (torch.zeros(1, s, device=dev) for _ in range(3))
    seed_m = torch.zeros(1, d * d, device=dev)
    seed_s = torch.zeros(1, d * d, device=dev)
    for si in range(nck - 2, -1, -1):
        t0, t1 = bounds[si], bounds[si + 1]
        L = t1 - t0
        seg_m, seg_s, ytmp = f32(1, L + 1, d * d), f32(1, L + 1, d * d), f32(1, L, d)
        out_m, out_s = f32(1, d * d), f32(1, d * d)
        sl = lambda x: x[:, t0:t1].contiguous()
        if rule == "titans":
            D.call("titans_forward_f32_cuda", k_mem=sl(t["k"]), v_mem=sl(t["v"]), q_mem=sl(t["q"]),
                   alpha=sl(t["alpha"]), theta=sl(t["theta"]), eta=sl(t["eta"]),
                   m_initial=mck[si:si + 1].contiguous(), s_initial=sck[si:si + 1].contiguous(),
                   m_states=seg_m, s_states=seg_s, y=ytmp, seq_len=L, d=d, batch_size=1,
                   input_stride=L, m_stride=d * d, error_clip=0.0, m_norm_max=0.0)
            D.call("titans_backward_segment_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"],
                   alpha=t["alpha"], theta=t["theta"], eta=t["eta"], m_states=seg_m,
                   s_states=seg_s, d_y=t["dy"], d_m_seed=seed_m, d_s_seed=seed_s, d_k_mem=dk,
                   d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_theta=dth, d_eta=de, d_m_out=out_m,
                   d_s_out=out_s, t_start=t0, t_end=t1, d=d, batch_size=1, seq_len=s,
                   error_clip=0.0)
        elif rule == "delta":
            D.call("delta_forward_f32_cuda", k_mem=sl(t["k"]), v_mem=sl(t["v"]), q_mem=sl(t["q"]),
                   alpha=sl(t["alpha"]), theta=sl(t["theta"]),
                   m_initial=mck[si:si + 1].contiguous(), m_states=seg_m, y=ytmp, seq_len=L, d=d,
                   batch_size=1, input_stride=L, m_stride=d * d, error_clip=0.0, m_norm_max=0.0)
            D.call("delta_backward_segment_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"],
                   alpha=t["alpha"], theta=t["theta"], m_states=seg_m, d_y=t["dy"],
                   d_m_seed=seed_m, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_theta=dth,
                   d_m_out=out_m, t_start=t0, t_end=t1, d=d, batch_size=1, seq_len=s,
                   error_clip=0.0)
        else:
            D.call("hebbian_forward_f32_cuda", k_mem=sl(t["k"]), v_mem=sl(t["v"]),
                   q_mem=sl(t["q"]), alpha=sl(t["alpha"]), m_initial=mck[si:si + 1].contiguous(),
                   m_states=seg_m, y=ytmp, seq_len=L, d=d, batch_size=1, input_stride=L,
                   m_stride=d * d)
            D.call("hebbian_backward_segment_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"],
                   alpha=t["alpha"], m_states=seg_m, d_y=t["dy"], d_m_seed=seed_m, d_k_mem=dk,
                   d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_m_out=out_m, t_start=t0, t_end=t1, d=d,
                   batch_size=1, seq_len=s)
        seed_m, seed_s = out_m, out_s
    got = dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dth, d_eta=de, d_m_initial=seed_m,
               d_s_initial=seed_s)
    keys = ["d_k", "d_v", "d_q", "d_alpha", "d_m_initial"]
    if rule != "hebbian":
        keys.append("d_theta")
    if rule == "titans":
        keys += ["d_eta", "d_s_initial"]
    for key in keys:
        assert rel_err(_np(got[key]), w[key]) <= REL, key


@pytest.mark.parametrize("rule", [0, 1, 2])
@pytest.mark.parametrize("d,s,interval,n", [(64, 32, 8, 3), (64, 21, 4, 2), (16, 12, 5, 2),
                                            (32, 16, 16, 1)])
def test_recompute_training_pair_exact(D, orc, rule, d, s, interval, n):
    """nlh_rule_forward/backward: checkpoints + in-kernel recompute == full-trajectory math,
    with per-problem d_m_initial."""
    name = {0: "delta", 1: "titans", 2: "hebbian"}[rule]
    p = make_problem(orc, n, s, d, 1700 + d + s + rule, "rand")
    w = oracle_exact(orc, name, p)
    t = to_dev(p)
    mc, sc, y = D.rule_forward(rule, t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                               t["m0"], t["s0"], interval)
    assert rel_err(_np(y), w["y"]) <= REL
    g = D.rule_backward(rule, t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], mc, sc,
                        t["dy"], interval)
    keys = ["d_k", "d_v", "d_q", "d_alpha", "d_m_initial"]
    if rule != 2:
        keys.append("d_theta")
    if rule == 1:
        keys += ["d_eta", "d_s_initial"]
    for key in keys:
        assert rel_err(_np(g[key]), w[key]) <= REL, key


@pytest.mark.parametrize("d,s,chunk,n", [(64, 48, 16, 2), (64, 20, 8, 3)])
def test_recompute_training_pair_frozen(D, orc, d, s, chunk, n):
    p = make_problem(orc, n, s, d, 1900 + d + s, "rand")
    w = oracle_chunkwise(orc, "titans", p, chunk)
    t = to_dev(p)
    mc, sc, y = D.rule_forward(1, t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                               t["m0"], t["s0"], chunk, chunk)
    assert rel_err(_np(y), w["y"]) <= REL
    g = D.rule_backward(1, t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], mc, sc,
                        t["dy"], chunk, chunk)
    for key in ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta", "d_m_initial", "d_s_initial"]:
        assert rel_err(_np(g[key]), w[key]) <= REL, key


@pytest.mark.parametrize("d,s,chunk,n", [(64, 64, 8, 3), (64, 8, 8, 2), (64, 37, 8, 2), (64, 50, 4, 1),
                                         (64, 21, 2, 2), (32, 40, 8, 2), (64, 130, 16, 1), (64, 9, 3, 2)])
def test_frozen_pair_on_a_full_trajectory(D, orc, d, s, chunk, n):
    """Frozen-M0 chunkwise Titans with every state stored (nlh_rule_forward / _backward with
    interval = 1): outputs, stored states at the chunk boundaries and every gradient against the
    oracle's chunkwise rule; ragged last chunks, chunks shorter than the prefetch pipeline and a
    single-chunk sequence included."""
    p = make_problem(orc, n, s, d, 2100 + d + s + chunk, "rand")
    w = oracle_chunkwise(orc, "titans", p, chunk)
    t = to_dev(p)
    ms, y = D.titans_frozen_stream_forward(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                                           t["m0"], t["s0"], chunk)
    assert rel_err(_np(y), w["y"]) <= REL
    nc = (s + chunk - 1) // chunk
    bounds = [min(c * chunk, s) for c in range(nc + 1)]
    assert rel_err(_np(ms[:, bounds]), w["m_chunk_states"].reshape(n, nc + 1, d * d)) <= REL
    g = D.titans_frozen_stream_backward(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], ms,
                                        t["dy"], chunk)
    for key in ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"]:
        assert rel_err(_np(g[key]), w[key]) <= REL, key
    for key in ["d_m_initial", "d_s_initial"]:            # per problem, like the oracle's
        assert rel_err(_np(g[key]), w[key].reshape(n, d * d)) <= REL, key
    g2 = D.titans_frozen_stream_backward(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], ms,
                                         t["dy"], chunk, want_initial=False)
    assert g2["d_m_initial"] is None and rel_err(_np(g2["d_k"]), w["d_k"]) <= REL


def test_input_stride_and_m_stride(D, orc):
    """Forward entries address batch element b at b*input_stride tokens and b*m_stride floats
    (core/kernels/titans_forward.cu:102-113): run on a sub-range of a longer padded buffer."""
    import torch
    n, s_full, s, d = 2, 24, 16, 64
    p = make_problem(orc, n, s_full, d, 2100, "rand")
    sub = {k_: (v_[:, :s] if v_.ndim >= 2 and v_.shape[1] == s_full else v_) for k_, v_ in p.items()}
    w = oracle_exact(orc, "titans", {k_: np.ascontiguousarray(v_) for k_, v_ in sub.items()})
    t = to_dev(p)
    m_pad = torch.zeros(n, 3 * d * d, device="cuda")
    s_pad = torch.zeros(n, 3 * d * d, device="cuda")
    m_pad[:, : d * d] = t["m0"]
    s_pad[:, : d * d] = t["s0"]
    ms = torch.empty(n, s + 1, d * d, device="cuda")
    ss = torch.empty(n, s + 1, d * d, device="cuda")
    y = torch.empty(n, s, d, device="cuda")
    D.call("titans_forward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
           theta=t["theta"], eta=t["eta"], m_initial=m_pad, s_initial=s_pad, m_states=ms,
           s_states=ss, y=y, seq_len=s, d=d, batch_size=n, input_stride=s_full,
           m_stride=3 * d * d, error_clip=0.0, m_norm_max=0.0)
    assert rel_err(_np(y), w["y"]) <= REL and rel_err(_np(ms), w["m_states"]) <= REL


def test_fused_forward(D, orc):
    """titans/dgd fused forward: in-place L2 norm of k,q + gates + recurrence
    (core/kernels/titans_forward.cu:492-742)."""
    import torch
    n, s, d = 2, 12, 64
    raw = make_problem(orc, n, s, d, 2300, "const", scale=0.5)
    w_a, w_t, w_e = (orc.rand_buf(2 * d, 2310 + i, 0.2) for i in range(3))
    b_a, b_t, b_e = 3.0, -4.6, 1.5   # level-0 gate biases (core/src/model.rs:1081-1122)
    kn, vv, qn = raw["k"].copy(), raw["v"], raw["q"].copy()
    gates = {}
    knorm = np.zeros((n, s), np.float32); qnorm = np.zeros((n, s), np.float32)
    for b in range(n):
        kn[b], knorm[b] = orc.l2_normalize_rows(raw["k"][b])
        qn[b], qnorm[b] = orc.l2_normalize_rows(raw["q"][b])
    for name, wv, bv, which, lo, hi in (("alpha", w_a, b_a, 0, 0.01, 0.99),
                                        ("theta", w_t, b_t, 1, 0.001, 0.5), ("eta", w_e, b_e, 0, 0, 0)):
        gates[name] = np.stack([orc.gate(kn[b], vv[b], wv, bv, which, lo, hi, name != "eta")[1]
                                for b in range(n)])
    p = dict(raw, k=kn, q=qn, **gates)
    w = oracle_exact(orc, "titans", p)
    t = to_dev(raw)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    kd, qd = t["k"].clone(), t["q"].clone()
    ms = torch.empty(n, s + 1, d * d, device="cuda"); ss = torch.empty_like(ms)
    y = torch.empty(n, s, d, device="cuda")
    outs = [torch.empty(n, s, device="cuda") for _ in range(5)]
    D.call("titans_fused_forward_f32_cuda", k_mem=kd, v_mem=t["v"], q_mem=qd, w_alpha=dev(w_a),
           b_alpha_ptr=dev([b_a]), w_theta=dev(w_t), b_theta_ptr=dev([b_t]), w_eta=dev(w_e),
           b_eta_ptr=dev([b_e]), alpha_floor=0.01, alpha_ceil=0.99, theta_floor=0.001,
           theta_ceil=0.5, m_initial=t["m0"], s_initial=t["s0"], m_states=ms, s_states=ss, y=y,
           alpha_out=outs[0], theta_out=outs[1], eta_out=outs[2], k_norms_out=outs[3],
           q_norms_out=outs[4], seq_len=s, d=d, batch_size=n, error_clip=0.0, m_norm_max=0.0)
    assert rel_err(_np(kd), kn) <= 1e-5 and rel_err(_np(qd), qn) <= 1e-5
    assert rel_err(_np(outs[3]), knorm) <= 1e-5 and rel_err(_np(outs[4]), qnorm) <= 1e-5
    for i, name in enumerate(("alpha", "theta", "eta")):
        assert rel_err(_np(outs[i]), gates[name]) <= 1e-5, name
    assert rel_err(_np(y), w["y"]) <= REL and rel_err(_np(ms), w["m_states"]) <= REL

    # DGD twin
    wd = oracle_exact(orc, "delta", p)
    kd, qd = t["k"].clone(), t["q"].clone()
    D.call("dgd_fused_forward_f32_cuda", k_mem=kd, v_mem=t["v"], q_mem=qd, w_alpha=dev(w_a),
           b_alpha_ptr=dev([b_a]), w_theta=dev(w_t), b_theta_ptr=dev([b_t]), alpha_floor=0.01,
           alpha_ceil=0.99, theta_floor=0.001, theta_ceil=0.5, m_initial=t["m0"], m_states=ms,
           y=y, alpha_out=outs[0], theta_out=outs[1], k_norms_out=outs[3], q_norms_out=outs[4],
           seq_len=s, d=d, batch_size=n, error_clip=0.0)
    assert rel_err(_np(y), wd["y"]) <= REL and rel_err(_np(ms), wd["m_states"]) <= REL


@pytest.mark.parametrize("rule", ["titans", "delta"])
def test_phase2_entries(D, orc, rule):
    """Per-chunk phase-2 kernels fed with externally computed errors reproduce the
    single-launch chunkwise kernels (core/src/dispatch.rs:2608-2680, 2783-2878)."""
    import torch
    n, s, d, chunk = 2, 20, 16, 8
    p = make_problem(orc, n, s, d, 2500, "rand")
    w = oracle_chunkwise(orc, rule, p, chunk)
    t = to_dev(p)
    nc = (s + chunk - 1) // chunk
    dev = t["k"].device
    f32 = lambda *sh: torch.zeros(*sh, dtype=torch.float32, device=dev)
    m_work, s_work = t["m0"].clone(), t["s0"].clone()
    mcs, scs, y = f32(n, nc + 1, d * d), f32(n, nc + 1, d * d), f32(n, s, d)
    for c in range(nc):
        t0, t1 = c * chunk, min((c + 1) * chunk, s)
        # phase 1 on the host side of the test: errors = M0 k - v (what cuBLAS + the epilogue produce)
        M0 = m_work.view(n, d, d)
        pred = torch.einsum("nij,ntj->nti", M0, t["k"][:, t0:t1])
        err = f32(n, chunk, d)
        err[:, : t1 - t0] = pred
        for b in range(n):
            D.call("error_subtract_clip_f32_cuda", predictions=err[b],
                   v=t["v"][b, t0:t1].contiguous(), total_rows=t1 - t0, d=d, error_clip=0.0)
        if rule == "titans":
            D.call("titans_phase2_forward_f32_cuda", k_mem=t["k"], q_mem=t["q"], alpha=t["alpha"],
                   theta=t["theta"], eta=t["eta"], errors=err, m_work=m_work, s_work=s_work,
                   m_chunk_states=mcs, s_chunk_states=scs, y=y, seq_len=s, d=d, batch_size=n,
                   chunk_size=chunk, chunk_idx=c, m_norm_max=0.0)
        else:
            D.call("delta_phase2_forward_f32_cuda", k_mem=t["k"], q_mem=t["q"], alpha=t["alpha"],
                   theta=t["theta"], errors=err, m_work=m_work, m_chunk_states=mcs, y=y,
                   seq_len=s, d=d, batch_size=n, chunk_size=chunk, chunk_idx=c, m_norm_max=0.0)
    assert rel_err(_np(y), w["y"]) <= REL and rel_err(_np(mcs), w["m_chunk_states"]) <= REL

    dk, dv, dq = f32(n, s, d), f32(n, s, d), f32(n, s, d)
    da, dth, de = f32(n, s), f32(n, s), f32(n, s)
    dM, dS, dM0 = f32(n, d * d), f32(n, d * d), f32(n, d * d)
    mrec, srec = f32(n, chunk + 1, d * d), f32(n, chunk + 1, d * d)
    for c in range(nc - 1, -1, -1):
        t0, t1 = c * chunk, min((c + 1) * chunk, s)
        M0 = mcs[:, c].reshape(n, d, d)
        err = f32(n, chunk, d)
        err[:, : t1 - t0] = torch.einsum("nij,ntj->nti", M0, t["k"][:, t0:t1]) - t["v"][:, t0:t1]
        if rule == "titans":
            D.call("titans_phase2_backward_f32_cuda", k_mem=t["k"], q_mem=t["q"], alpha=t["alpha"],
                   theta=t["theta"], eta=t["eta"], errors=err, m_chunk_states=mcs,
                   s_chunk_states=scs, d_y=t["dy"], d_k_mem=dk, d_v_mem=dv, d_q_mem=dq,
                   d_alpha=da, d_theta=dth, d_eta=de, d_M=dM, d_S=dS, d_M0=dM0, m_recompute=mrec,
                   s_recompute=srec, seq_len=s, d=d, batch_size=n, chunk_size=chunk, chunk_idx=c,
                   m_norm_max=0.0)
        else:
            D.call("delta_phase2_backward_f32_cuda", k_mem=t["k"], q_mem=t["q"], alpha=t["alpha"],
                   theta=t["theta"], errors=err, m_chunk_states=mcs, d_y=t["dy"], d_k_mem=dk,
                   d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_theta=dth, d_M=dM, d_M0=dM0,
                   m_recompute=mrec, seq_len=s, d=d, batch_size=n, chunk_size=chunk, chunk_idx=c,
                   m_norm_max=0.0)
    got = dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dth, d_eta=de, d_m_initial=dM,
               d_s_initial=dS)
    keys = ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_m_initial"]
    if rule == "titans":
        keys += ["d_eta", "d_s_initial"]
    for key in keys:
        assert rel_err(_np(got[key]), w[key]) <= REL, key


def test_m_norm_clamp(D, orc):
    import torch
    d, n = 16, 3
    m = orc.rand_buf(n * d * d, 2700, 1.0).reshape(n, d * d)
    want = orc.m_norm_clamp(m, d, n, 2.0)
    t = torch.from_numpy(m.copy()).cuda()
    D.call("m_norm_clamp_batch_f32_cuda", m=t, d=d, batch_size=n, m_norm_max=2.0)
    assert rel_err(_np(t), want) <= 1e-6
    t1 = torch.from_numpy(m[0].copy()).cuda()
    D.call("m_norm_clamp_f32_cuda", m=t1, d=d, m_norm_max=2.0)
    assert rel_err(_np(t1), want[0]) <= 1e-6
    t2 = torch.from_numpy(m.copy()).cuda()
    D.call("m_norm_clamp_batch_f32_cuda", m=t2, d=d, batch_size=n, m_norm_max=0.0)   # disabled
    assert np.array_equal(_np(t2), m)


def test_empty_and_invalid_inputs(D):
    import torch
    from nl_hecate_b200 import ffi
    z = torch.zeros(4, device="cuda")
    # batch_size = 0: nothing is launched and no error is recorded
    D.call("titans_forward_f32_cuda", k_mem=z, v_mem=z, q_mem=z, alpha=z, theta=z, eta=z,
           m_initial=z, s_initial=z, m_states=z, s_states=z, y=z, seq_len=4, d=8, batch_size=0,
           input_stride=4, m_stride=64, error_clip=0.0, m_norm_max=0.0)
    # d <= 0 is rejected with a recorded error instead of the reference's exit(1)
    with pytest.raises(RuntimeError):
        D.call("titans_forward_f32_cuda", k_mem=z, v_mem=z, q_mem=z, alpha=z, theta=z, eta=z,
               m_initial=z, s_initial=z, m_states=z, s_states=z, y=z, seq_len=4, d=0,
               batch_size=1, input_stride=4, m_stride=64, error_clip=0.0, m_norm_max=0.0)
    with pytest.raises(RuntimeError):
        D.call("titans_chunkwise_forward_f32_cuda", k_mem=z, v_mem=z, q_mem=z, alpha=z, theta=z,
               eta=z, m_initial=z, s_initial=z, m_chunk_states=z, s_chunk_states=z, y=z,
               seq_len=4, d=8, batch_size=1, chunk_size=0, error_clip=0.0, m_norm_max=0.0)
    assert ffi.lib().nlh_last_status() == 0   # cleared by the wrapper after raising


@pytest.mark.parametrize("d,s,n", [(64, 40, 3), (32, 17, 2), (64, 1, 1)])
def test_titans_exact_without_momentum_trajectory(D, orc, d, s, n):
    """s_states = NULL: forward stores only M; backward derives S_t from consecutive M states
    (d_eta = (<M_{t+1} - (1-alpha) M_t, dS> + theta e.(dS k)) / eta)."""
    p = make_problem(orc, n, s, d, 2900 + d + s, "rand")
    w = oracle_exact(orc, "titans", p)
    t = to_dev(p)
    ms, ss, y = D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                                    t["m0"], t["s0"], store_s=False)
    assert ss is None
    assert rel_err(_np(y), w["y"]) <= REL and rel_err(_np(ms), w["m_states"]) <= REL
    g = D.titans_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], ms, None,
                             t["dy"])
    _check_bwd(g, w, ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta", "d_m_initial",
                      "d_s_initial"])


@pytest.mark.parametrize("n,s", [(3, 40), (1, 9), (6, 130)])
def test_row_split_exact_pair_matches_one_cta_per_problem(D, orc, n, s):
    """With no more problems than SMs the exact head_dim-64 kernels divide every problem's rows over
    two CTAs (option NLH_OPT_ROW_SPLIT, default on); the M-only backward then adds two partial sums
    into d_q, d_k and the gate gradients, which it zeroes itself. Both modes against the oracle, with
    the outputs pre-filled with garbage in split mode (nothing may depend on the caller's zeroing)."""
    import torch
    p = make_problem(orc, n, s, 64, 5200 + n + s, "rand")
    w = oracle_exact(orc, "titans", p)
    t = to_dev(p)
    for on in (1, 0):
        D.call("nlh_set_option", option=3, value=on)
        try:
            ms, ss, y = D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                                            t["m0"], t["s0"], store_s=False)
            assert rel_err(_np(y), w["y"]) <= REL and rel_err(_np(ms), w["m_states"]) <= REL
            ms2, ss2, y2 = D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"],
                                               t["m0"], t["s0"])
            assert rel_err(_np(ss2), w["s_states"]) <= REL and torch.equal(y, y2)
            nan = lambda like: torch.full_like(like, float("nan"))
            g = dict(d_k=nan(t["k"]), d_v=nan(t["k"]), d_q=nan(t["k"]), d_alpha=nan(t["alpha"]),
                     d_theta=nan(t["alpha"]), d_eta=nan(t["alpha"]),
                     d_m_initial=torch.zeros(64 * 64, device="cuda"), d_s_initial=torch.zeros(64 * 64, device="cuda"))
            if not on:   # one CTA per problem follows the drop-in contract: d_k, d_v, d_q pre-zeroed
                for key in ("d_k", "d_v", "d_q"):
                    g[key].zero_()
            D.call("titans_backward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
                   theta=t["theta"], eta=t["eta"], m_states=ms, s_states=None, d_y=t["dy"], d_k_mem=g["d_k"],
                   d_v_mem=g["d_v"], d_q_mem=g["d_q"], d_alpha=g["d_alpha"], d_theta=g["d_theta"],
                   d_eta=g["d_eta"], d_m_initial=g["d_m_initial"], d_s_initial=g["d_s_initial"], seq_len=s,
                   d=64, batch_size=n, error_clip=0.0)
        finally:
            D.call("nlh_set_option", option=3, value=1)
        _check_bwd(g, w, ["d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta", "d_m_initial", "d_s_initial"])


@pytest.mark.parametrize("d,s,n", [(64, 5, 2), (64, 16, 3), (64, 37, 3), (32, 130, 2), (64, 130, 150)])
def test_bulk_staged_forward_equals_cp_async_staging(D, orc, d, s, n):
    """NLH_OPT_BULK_STAGING: the register-resident forward kernels stage the k, v, q tiles with one
    bulk asynchronous copy per stream and tile, completion counted on an mbarrier (default on). The
    staging does not touch the arithmetic: every rule's outputs are bit-identical to the cp.async
    staging, on whole, ragged and single tiles, exact and frozen, and no bounded wait ran out."""
    import torch
    p = make_problem(orc, n, s, d, 7100 + d + s + n, "rand")
    t = to_dev(p)
    outs = {}
    D.call("nlh_set_option", option=3, value=0)      # one CTA per problem at every n
    D.call("nlh_set_option", option=2, value=0)      # frozen rules on the per-token kernels
    try:
        for on in (1, 0):
            D.call("nlh_set_option", option=5, value=on)
            o = []
            o += D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], t["m0"], t["s0"])
            o += D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], t["m0"], t["s0"],
                                     store_s=False)[::2]
            o += D.delta_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["m0"])
            o += D.hebbian_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["m0"])
            o += D.titans_chunkwise_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], t["m0"],
                                               t["s0"], 8)
            o += D.delta_chunkwise_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["m0"], 8)
            o += D.titans_frozen_stream_forward(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], t["m0"],
                                                t["s0"], 8)
            outs[on] = o
    finally:
        for opt in (2, 3, 5):
            D.call("nlh_set_option", option=opt, value=1)
    assert len(outs[1]) == len(outs[0])
    for a, b in zip(outs[1], outs[0]):
        assert a.shape == b.shape and torch.equal(a, b)
    assert D.ffi.lib().nlh_bulk_timeout_flag() == 0
    if n <= 3:
        w = oracle_exact(orc, "titans", p)
        assert rel_err(_np(outs[1][0]), w["m_states"]) <= REL and rel_err(_np(outs[1][2]), w["y"]) <= REL


def test_null_momentum_trajectory_rejected_off_the_fast_path(D, orc):
    p = make_problem(orc, 1, 6, 16, 2990, "rand")   # d = 16 runs the generic kernels
    t = to_dev(p)
    with pytest.raises(RuntimeError, match="register-resident"):
        D.titans_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], t["m0"],
                            t["s0"], store_s=False)


def test_kernels_reproduce_the_committed_small_vectors(D, orc):
    """The committed known-answer file (tests/golden/oracle_small.npz, frozen oracle outputs on
    the reference's rand_buf inputs) against the CUDA kernels: Titans exact pair at d=8, s=6."""
    import os
    import torch
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_small.npz"))
    d, s = 8, 6
    r = lambda n, seed: orc.rand_buf(n, seed, 0.1)
    k, v, q, dy = (torch.from_numpy(r(s * d, 100 + i).reshape(1, s, d)).cuda() for i in range(4))
    m0 = torch.from_numpy(r(d * d, 104).reshape(1, d * d)).cuda()
    s0 = torch.from_numpy(r(d * d, 105).reshape(1, d * d)).cuda()
    al = torch.full((1, s), 0.05, device="cuda")
    th = torch.full((1, s), 0.01, device="cuda")
    et = torch.full((1, s), 0.9, device="cuda")
    ms, ss, y = D.titans_forward_dd(k, v, q, al, th, et, m0, s0)
    assert max_abs(_np(y[0]), g["titans_y"]) < 1e-6
    assert max_abs(_np(ms[0, -1]), g["titans_m_final"]) < 1e-6
    got = D.titans_backward_dd(k, v, q, al, th, et, ms, ss, dy)
    for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"):
        assert rel_err(_np(got[key][0]), g["titans_" + key]) <= REL, key
