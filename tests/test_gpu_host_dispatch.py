"""GPU: the compiled host-slice dispatch layer (nlh_*_dispatch, host arrays in and out) vs the
CPU oracle, in the style of the reference's kernel tests (core/tests/test_cuda_titans.rs:69-340:
rand_buf inputs, forward max-abs 1e-5, backward 1e-4)."""
import numpy as np
import pytest

from helpers import make_problem, max_abs, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def D():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch
    return dispatch


def _one(p):
    return {k: v[0] for k, v in p.items()}


@pytest.mark.parametrize("d,s", [(64, 20), (8, 7)])
def test_titans_host_dispatch(D, orc, d, s):
    p = _one(make_problem(orc, 1, s, d, 4100 + d, "const"))
    f = orc.titans_forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"])
    got = D.host_rule_forward("titans", p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], p["m0"], p["s0"])
    assert max_abs(got["y"], f["y"]) < 1e-5 and max_abs(got["m_states"], f["m_states"]) < 1e-5
    assert max_abs(got["s_states"], f["s_states"]) < 1e-5
    want = orc.titans_backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["eta"], f["m_states"],
                               f["s_states"], p["dy"])
    g = D.host_rule_backward("titans", p["k"], p["v"], p["q"], p["alpha"], got["m_states"], p["dy"],
                             theta=p["theta"], eta=p["eta"], s_states=got["s_states"])
    for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta", "d_m_initial", "d_s_initial"):
        assert max_abs(g[key], np.asarray(want[key]).reshape(g[key].shape)) < 1e-4, key


@pytest.mark.parametrize("rule", ["delta", "dgd", "hebbian"])
def test_delta_dgd_hebbian_host_dispatch(D, orc, rule):
    d, s = 32, 11
    p = _one(make_problem(orc, 1, s, d, 4200, "rand"))
    if rule == "hebbian":
        f = orc.hebbian_forward(p["k"], p["v"], p["q"], p["alpha"], p["m0"])
        want = orc.hebbian_backward(p["k"], p["v"], p["q"], p["alpha"], f["m_states"], p["dy"])
        got = D.host_rule_forward("hebbian", p["k"], p["v"], p["q"], p["alpha"], m0=p["m0"])
        g = D.host_rule_backward("hebbian", p["k"], p["v"], p["q"], p["alpha"], got["m_states"], p["dy"])
    else:
        f = orc.delta_forward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], p["m0"])
        want = orc.delta_backward(p["k"], p["v"], p["q"], p["alpha"], p["theta"], f["m_states"], p["dy"])
        got = D.host_rule_forward(rule, p["k"], p["v"], p["q"], p["alpha"], theta=p["theta"], m0=p["m0"])
        g = D.host_rule_backward(rule, p["k"], p["v"], p["q"], p["alpha"], got["m_states"], p["dy"],
                                 theta=p["theta"])
    assert rel_err(got["y"], f["y"]) <= 1e-4 and rel_err(got["m_states"], f["m_states"]) <= 1e-4
    for key in g:
        assert rel_err(g[key], np.asarray(want[key]).reshape(g[key].shape)) <= 1e-4, key


def test_swa_host_dispatch(D, orc):
    s, nh, hd, w = 80, 2, 32, 24
    n = s * nh * hd
    q, k, v = (orc.bf16_round(orc.rand_buf(n, 4300 + i, 0.5)).reshape(s, nh * hd) for i in range(3))
    d_out = orc.rand_buf(n, 4303, 1.0).reshape(s, nh * hd)
    f = orc.swa_forward(q, k, v, nh, hd, w)
    want = orc.swa_backward(q, k, v, f["attn_weights"], d_out, nh, hd, w)
    got = D.host_swa_forward(q, k, v, nh, hd, w)
    assert max_abs(got["out"], f["out"]) < 1e-2
    assert max_abs(got["attn_weights"], f["attn_weights"]) < 1e-2
    g = D.host_swa_backward(q, k, v, None, d_out, nh, hd, w)
    for key in ("d_q", "d_k", "d_v"):
        assert rel_err(g[key], want[key]) <= 2e-2, key


def test_host_dispatch_rejects_bad_arguments(D):
    z = np.zeros((4, 8), np.float32)
    with pytest.raises(RuntimeError):
        D.call("nlh_delta_forward_dispatch", k_mem=None, v_mem=None, q_mem=None, alpha=None, theta=None,
               m_initial=None, m_states=None, y=None, seq_len=4, d=8, error_clip=0.0, m_norm_max=0.0)
    with pytest.raises(RuntimeError):
        D.call("nlh_swa_forward_dispatch", q=D._hp(z), k=D._hp(z), v=D._hp(z), out=D._hp(z), attn_weights=None,
               seq_len=0, num_heads=1, head_dim=8, window_size=4)
