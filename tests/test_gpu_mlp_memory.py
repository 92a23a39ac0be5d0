"""Titans LMM with a two-layer MLP memory: the CUDA pair behind titans_mlp_forward_f32_cuda /
titans_mlp_backward_f32_cuda against the CPU oracle (oracle/mlp_memory.py, a restatement of
TitansLMM::step_mlp / step_backward_mlp, core/src/titans_lmm.rs:653-1131) on the same seeded
inputs. fp32; tolerance 1e-5 relative to the largest magnitude of each output (1e-4 for the
gradients, whose sums run over the whole packed state)."""
import numpy as np
import pytest

from helpers import rel_err

pytestmark = pytest.mark.gpu
REL_FWD, REL_BWD = 1e-5, 1e-4


@pytest.fixture(scope="module")
def D():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import nl_hecate_b200.dispatch as disp
    return disp


def _dev(p):
    import torch
    return {k: torch.from_numpy(v).cuda() for k, v in p.items()}


def _np(t):
    return t.detach().cpu().numpy()


def _pair(D, mlp, n, s, d, dh, act, seed, m_norm_max=0.0, state_scale=0.1, s0=False):
    p = mlp.make_problem(n, s, d, dh, seed, np.float32, state_scale=state_scale)
    if s0:
        p["s0"] = (np.random.default_rng(seed + 1).standard_normal(p["s0"].shape) * 0.02).astype(np.float32)
    wm, ws, wy = mlp.forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], dh, act,
                             m_norm_max)
    wg = mlp.backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], wm, ws, p["dy"], dh, act)
    t = _dev(p)
    ms, ss, y = D.titans_mlp_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], t["m0"], t["s0"],
                                        dh, act, m_norm_max)
    assert rel_err(_np(y), wy) <= REL_FWD
    assert rel_err(_np(ms), wm) <= REL_FWD and rel_err(_np(ss), ws) <= REL_FWD
    g = D.titans_mlp_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], ms, ss, t["dy"], dh, act)
    for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"):
        assert rel_err(_np(g[key]), wg[key]) <= REL_BWD, key
    for key in ("d_m_initial", "d_s_initial"):          # the entry adds them over the batch
        assert rel_err(_np(g[key]), wg[key].sum(axis=0)) <= REL_BWD, key
    return t, ms, ss, y, g


@pytest.mark.parametrize("act", [0, 1, 2])
@pytest.mark.parametrize("n,s,d,dh", [(2, 9, 64, 256), (3, 12, 32, 128), (1, 1, 64, 256), (2, 7, 8, 32),
                                      (2, 6, 24, 40), (1, 5, 64, 128), (5, 4, 16, 16)])
def test_pair_matches_the_oracle(D, act, n, s, d, dh):
    """Head sizes of the reference's configs (d 64, expansion 4) and of its tests (d 8), sizes that
    are no power of two, one-token sequences, all three activations, carried momentum."""
    from oracle import mlp_memory as mlp
    _pair(D, mlp, n, s, d, dh, act, 100 * act + n + s + d, s0=(n % 2 == 0))


def test_long_sequence_and_many_problems(D):
    """More problems than SMs and a 96-token recurrence at the largest supported state."""
    from oracle import mlp_memory as mlp
    _pair(D, mlp, 160, 3, 64, 256, 0, 900)
    _pair(D, mlp, 1, 96, 64, 256, 0, 901, s0=True)


def test_frobenius_projection(D):
    """m_norm_max bounds every stored state; the backward passes straight through (the oracle's
    backward on the projected trajectory)."""
    from oracle import mlp_memory as mlp
    t, ms, ss, y, g = _pair(D, mlp, 2, 8, 32, 128, 0, 950, m_norm_max=2.0, state_scale=0.3)
    import torch
    assert float(torch.linalg.vector_norm(ms[:, 1:], dim=-1).max()) <= 2.0 * (1 + 1e-5)
    free = D.titans_mlp_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], t["m0"], t["s0"], 128)[0]
    assert float(torch.linalg.vector_norm(free[:, 1:], dim=-1).max()) > 2.0


def test_backward_adds_initial_state_gradients_and_overwrites_the_rest(D):
    """The drop-in contract of titans_mlp_backward_f32_cuda: d_m_initial / d_s_initial accumulate
    (atomicAdd over the batch into caller-zeroed buffers), every other output is written whatever
    it held."""
    import torch
    from oracle import mlp_memory as mlp
    n, s, d, dh = 3, 5, 32, 128
    t, ms, ss, y, g = _pair(D, mlp, n, s, d, dh, 1, 960)
    ssz = D.mlp_state_size(d, dh)
    nan = lambda like: torch.full_like(like, float("nan"))
    out = dict(d_k_mem=nan(t["k"]), d_v_mem=nan(t["k"]), d_q_mem=nan(t["k"]), d_alpha=nan(t["alpha"]),
               d_theta=nan(t["alpha"]), d_eta=nan(t["alpha"]), d_m_initial=torch.ones(ssz, device="cuda"),
               d_s_initial=torch.ones(ssz, device="cuda"))
    D.call("titans_mlp_backward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
           theta=t["theta"], eta=t["eta"], m_states=ms, s_states=ss, d_y=t["dy"], seq_len=s, d=d, d_hidden=dh,
           batch_size=n, input_stride=s * d, m_stride=(s + 1) * ssz, activation=1, m_norm_max=0.0, **out)
    assert torch.equal(out["d_k_mem"], g["d_k"]) and torch.equal(out["d_alpha"], g["d_alpha"])
    assert rel_err(_np(out["d_m_initial"] - 1.0), _np(g["d_m_initial"])) <= 1e-5
    assert rel_err(_np(out["d_s_initial"] - 1.0), _np(g["d_s_initial"])) <= 1e-5


def test_unsupported_and_invalid_shapes_launch_nothing(D):
    import torch
    z = torch.zeros(4, device="cuda")
    kw = dict(k_mem=z, v_mem=z, q_mem=z, alpha=z, theta=z, eta=z, m_initial=z, s_initial=z, m_states=z, s_states=z,
              y=z, seq_len=1, batch_size=1, input_stride=1, m_stride=1, m_norm_max=0.0)
    with pytest.raises(RuntimeError, match="does not fit|not supported"):
        D.call("titans_mlp_forward_f32_cuda", d=128, d_hidden=512, activation=0, **kw)
    with pytest.raises(RuntimeError, match="activation"):
        D.call("titans_mlp_forward_f32_cuda", d=4, d_hidden=8, activation=3, **kw)
    D.call("titans_mlp_forward_f32_cuda", d=4, d_hidden=8, activation=0, **{**kw, "batch_size": 0})


def test_host_slice_entries_match_the_oracle(D):
    """nlh_titans_mlp_{forward,backward}_dispatch: the compiled counterpart of the reference's
    titans_mlp_forward_cuda / titans_mlp_backward_cuda (core/src/dispatch.rs:897-1070) — host arrays
    in and out, a batch of problems."""
    from oracle import mlp_memory as mlp
    n, s, d, dh = 3, 7, 64, 256
    p = mlp.make_problem(n, s, d, dh, 990)
    wm, ws, wy = mlp.forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], dh, 1)
    wg = mlp.backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], wm, ws, p["dy"], dh, 1)
    f, g = D.host_titans_mlp_pair(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], p["dy"],
                                  dh, activation=1)
    assert rel_err(f["y"], wy) <= REL_FWD and rel_err(f["m_states"], wm) <= REL_FWD and rel_err(f["s_states"], ws) <= REL_FWD
    for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"):
        assert rel_err(g[key], wg[key]) <= REL_BWD, key
    for key in ("d_m_initial", "d_s_initial"):
        assert rel_err(g[key], wg[key].sum(axis=0)) <= REL_BWD, key
    with pytest.raises(RuntimeError):
        D.host_titans_mlp_pair(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"], p["dy"],
                               dh, activation=7)


def test_unaligned_state_buffers_take_the_generic_kernels(D):
    """The float4 kernels of head 64 / hidden 256 need 16-byte aligned state buffers; with a
    trajectory that starts 4 bytes off the library runs the generic kernels instead — same results."""
    import torch
    from oracle import mlp_memory as mlp
    n, s, d, dh = 2, 5, 64, 256
    t, ms, ss, y, g = _pair(D, mlp, n, s, d, dh, 0, 970)
    ssz = D.mlp_state_size(d, dh)
    raw_m = torch.empty(n * (s + 1) * ssz + 1, device="cuda")
    raw_s = torch.empty(n * (s + 1) * ssz + 1, device="cuda")
    ms2, ss2 = raw_m[1:], raw_s[1:]
    assert ms2.data_ptr() % 16 == 4
    y2 = torch.empty_like(y)
    D.call("titans_mlp_forward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"], theta=t["theta"],
           eta=t["eta"], m_initial=t["m0"], s_initial=t["s0"], m_states=ms2.data_ptr(), s_states=ss2.data_ptr(), y=y2,
           seq_len=s, d=d, d_hidden=dh, batch_size=n, input_stride=s * d, m_stride=(s + 1) * ssz, activation=0,
           m_norm_max=0.0)
    assert rel_err(_np(y2), _np(y)) <= 1e-6 and rel_err(_np(ms2), _np(ms).ravel()) <= 1e-6
    out = {k_: torch.empty_like(t["k"]) for k_ in ("d_k_mem", "d_v_mem", "d_q_mem")}
    out.update({k_: torch.empty_like(t["alpha"]) for k_ in ("d_alpha", "d_theta", "d_eta")})
    out.update(d_m_initial=torch.zeros(ssz, device="cuda"), d_s_initial=torch.zeros(ssz, device="cuda"))
    D.call("titans_mlp_backward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"], theta=t["theta"],
           eta=t["eta"], m_states=ms2.data_ptr(), s_states=ss2.data_ptr(), d_y=t["dy"], seq_len=s, d=d, d_hidden=dh,
           batch_size=n, input_stride=s * d, m_stride=(s + 1) * ssz, activation=0, m_norm_max=0.0, **out)
    for a_, b_ in (("d_k_mem", "d_k"), ("d_v_mem", "d_v"), ("d_q_mem", "d_q"), ("d_alpha", "d_alpha"),
                   ("d_theta", "d_theta"), ("d_eta", "d_eta"), ("d_m_initial", "d_m_initial")):
        assert rel_err(_np(out[a_]), _np(g[b_])) <= 1e-5, a_


def test_full_length_sequences_within_the_conditioning_of_each_problem(D):
    """512 tokens (the bench length) at head 64 / hidden 256, against the float64 oracle. With
    learning-rate gates around 0.015 (the scale of the reference's default gate bias) every problem
    is well conditioned and is held to the plain tolerances (1e-5 forward, 1e-4 backward). With
    gates four times larger the inner gradient descent of some problems is ill-conditioned over
    hundreds of tokens — the oracle in float32 and in float64 then drift apart by themselves — so
    there every problem is held to max(plain tolerance, 30 x the oracle's own float32-float64 gap)."""
    from oracle import mlp_memory as mlp
    n, s, d, dh = 4, 512, 64, 256
    for theta_scale in (0.25, 1.0):
        p = mlp.make_problem(n, s, d, dh, 4242)
        p["theta"] *= np.float32(theta_scale)
        p64 = {key: val.astype(np.float64) for key, val in p.items()}
        args = lambda q_: (q_["k"], q_["v"], q_["q"], q_["alpha"], q_["theta"], q_["eta"])
        m32, s32, y32 = mlp.forward(*args(p), p["m0"], p["s0"], dh, 0)
        m64, s64_, y64 = mlp.forward(*args(p64), p64["m0"], p64["s0"], dh, 0)
        g32 = mlp.backward(*args(p), m32, s32, p["dy"], dh, 0)
        g64 = mlp.backward(*args(p64), m64, s64_, p64["dy"], dh, 0)
        t = _dev(p)
        ms, ss, y = D.titans_mlp_forward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], t["m0"], t["s0"],
                                            dh, 0)
        g = D.titans_mlp_backward_dd(t["k"], t["v"], t["q"], t["alpha"], t["theta"], t["eta"], ms, ss, t["dy"], dh, 0)
        for b in range(n):
            gap = max(rel_err(m32[b], m64[b]), rel_err(y32[b], y64[b]))
            if theta_scale < 1.0:
                assert 30 * gap <= REL_FWD, (b, gap)        # well conditioned: the plain tolerance applies
            assert rel_err(_np(y[b]), y64[b]) <= max(REL_FWD, 30 * gap), (theta_scale, b, gap)
            assert rel_err(_np(ms[b]), m64[b]) <= max(REL_FWD, 30 * gap), (theta_scale, b, gap)
            for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"):
                ggap = max(gap, rel_err(g32[key][b], g64[key][b]))
                if theta_scale < 1.0:
                    assert 30 * ggap <= REL_BWD, (b, key, ggap)
                assert rel_err(_np(g[key][b]), g64[key][b]) <= max(REL_BWD, 30 * ggap), (theta_scale, b, key, ggap)
