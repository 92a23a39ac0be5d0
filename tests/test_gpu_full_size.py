"""GPU: memory-rule kernels at the benchmark shapes — size-independent properties over the WHOLE
batch (element-wise parity against the oracle on sampled problems at full length is in
test_gpu_baseline_shapes.py):
  * problems are independent: a problem run alone gives bit-identical results to the same
    problem inside the full batch (one CTA per problem, same instruction order; with the rows of
    a lone problem divided over two CTAs the column sums differ in the order of two partial sums);
  * the backward is linear in d_y;
  * the exact pair with the M-only trajectory (s_states = NULL) agrees with the pair that
    stores and reads the S trajectory (relative 1e-4: S is rebuilt from M differences);
  * chunk size 1 of the frozen rule equals the per-token rule.
Shapes: cfg2 (N = 128 problems, S = 2048, head_dim 64, chunk 64) and the stacked model's level
0 (N = 512, S = 512)."""
import numpy as np
import pytest

from helpers import max_abs, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def D():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch
    return dispatch


def _np(t):
    return t.detach().float().cpu().numpy()


def _problem(n, s, d=64, seed=0):
    import torch
    import torch.nn.functional as F
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *sh: torch.randn(*sh, device="cuda", generator=g)
    k, q, v = F.normalize(r(n, s, d), dim=-1), F.normalize(r(n, s, d), dim=-1), r(n, s, d) * 0.5
    alpha = torch.sigmoid(r(n, s) + 3).contiguous()
    theta = F.softplus(r(n, s) - 4.6).contiguous()
    eta = torch.sigmoid(r(n, s) + 1.5).contiguous()
    m0 = r(n, d * d) * 0.05
    s0 = torch.zeros(n, d * d, device="cuda")
    dy = r(n, s, d)
    return k, v, q, alpha, theta, eta, m0, s0, dy


def test_level0_exact_pair_properties(D):
    import torch
    n, s = 512, 512
    k, v, q, al, th, et, m0, s0, dy = _problem(n, s, seed=11)
    ms, _, y = D.titans_forward_dd(k, v, q, al, th, et, m0, s0, store_s=False)
    g = D.titans_backward_dd(k, v, q, al, th, et, ms, None, dy)
    # with the S trajectory stored and read
    ms2, ss2, y2 = D.titans_forward_dd(k, v, q, al, th, et, m0, s0, store_s=True)
    g2 = D.titans_backward_dd(k, v, q, al, th, et, ms2, ss2, dy)
    assert torch.equal(y, y2) and torch.equal(ms, ms2)
    for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"):
        assert rel_err(_np(g[key]), _np(g2[key])) <= 1e-4, key
    # a problem alone == the same problem inside the batch (forward and backward): bit for bit with
    # one CTA per problem; with the rows of a lone problem divided over two CTAs (the default below
    # the SM count) the forward is still bit-identical and the column sums of the backward differ
    # only in the order of two partial sums
    for i in (0, 300, 511):
        sl = slice(i, i + 1)
        one = [t[sl].contiguous() for t in (k, v, q, al, th, et, m0, s0, dy)]
        for split in (0, 1):
            D.call("nlh_set_option", option=3, value=split)
            try:
                ms1, _, y1 = D.titans_forward_dd(*one[:8], store_s=False)
                g1 = D.titans_backward_dd(*one[:6], ms1, None, one[8])
            finally:
                D.call("nlh_set_option", option=3, value=1)
            assert torch.equal(y1, y[sl]) and torch.equal(ms1, ms[sl])
            for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"):
                if split:
                    assert rel_err(_np(g1[key]), _np(g[key][sl])) <= 1e-5, key
                else:
                    assert torch.equal(g1[key], g[key][sl]), key
    # linearity of the backward in d_y
    gl = D.titans_backward_dd(k, v, q, al, th, et, ms, None, (2.0 * dy).contiguous())
    for key in ("d_k", "d_q", "d_alpha", "d_eta"):
        assert rel_err(_np(gl[key]), 2.0 * _np(g[key])) <= 1e-5, key
    assert np.isfinite(_np(g["d_m_initial"])).all()


def test_cfg2_chunkwise_pair_properties(D):
    import torch
    n, s, c = 128, 2048, 64
    k, v, q, al, th, et, m0, s0, dy = _problem(n, s, seed=12)
    mc, sc, y = D.titans_chunkwise_forward_dd(k, v, q, al, th, et, m0, s0, c)
    g = D.titans_chunkwise_backward_dd(k, v, q, al, th, et, mc, sc, dy, c)
    assert np.isfinite(_np(y)).all()
    for i in (0, 77, 127):
        sl = slice(i, i + 1)
        one = [t[sl].contiguous() for t in (k, v, q, al, th, et, m0, s0, dy)]
        mc1, sc1, y1 = D.titans_chunkwise_forward_dd(*one[:8], c)
        g1 = D.titans_chunkwise_backward_dd(*one[:6], mc1, sc1, one[8], c)
        assert torch.equal(y1, y[sl]) and torch.equal(mc1, mc[sl])
        for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"):
            assert torch.equal(g1[key], g[key][sl]), key
    gl = D.titans_chunkwise_backward_dd(k, v, q, al, th, et, mc, sc, (0.5 * dy).contiguous(), c)
    for key in ("d_k", "d_v", "d_q", "d_theta"):
        assert rel_err(_np(gl[key]), 0.5 * _np(g[key])) <= 1e-5, key


def test_chunk_one_equals_per_token_rule_at_length(D):
    import torch
    n, s = 16, 2048
    k, v, q, al, th, et, m0, s0, dy = _problem(n, s, seed=13)
    ms, ss, y = D.titans_forward_dd(k, v, q, al, th, et, m0, s0)
    mc, sc, yc = D.titans_chunkwise_forward_dd(k, v, q, al, th, et, m0, s0, 1)
    assert rel_err(_np(yc), _np(y)) <= 1e-4
    assert rel_err(_np(mc[:, -1]), _np(ms[:, -1])) <= 1e-4
    g = D.titans_backward_dd(k, v, q, al, th, et, ms, ss, dy)
    gc = D.titans_chunkwise_backward_dd(k, v, q, al, th, et, mc, sc, dy, 1)
    for key in ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_eta"):
        assert rel_err(_np(gc[key]), _np(g[key])) <= 1e-3, key
