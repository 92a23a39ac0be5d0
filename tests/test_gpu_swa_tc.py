"""GPU: the tcgen05/TMEM SWA forward (head_dim 64) vs the CPU oracle and vs the mma.sync kernel.
Relative error <= 2e-2 (bf16 tensor cores); the kernel's bounded-wait flag must stay clear."""
import numpy as np
import pytest

from helpers import max_abs, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture()
def tc_on():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch as D
    D.call("nlh_set_option", option=1, value=1)
    yield D
    D.call("nlh_set_option", option=1, value=1)   # the library default


def _np(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("b,s,nh,w,n_p", [(1, 128, 1, 128, 0), (1, 64, 1, 64, 0), (2, 300, 2, 96, 0),
                                          (1, 513, 2, 512, 0), (1, 200, 1, 40, 7), (1, 1, 1, 1, 0),
                                          (2, 1000, 1, 256, 0)])
def test_tcgen05_forward_matches_oracle(tc_on, orc, b, s, nh, w, n_p):
    import torch
    D = tc_on
    hd = 64
    shape = (b, s, nh * hd)
    mk = lambda sd: torch.from_numpy(orc.rand_buf(b * s * nh * hd, sd, 0.5).reshape(shape)).cuda().bfloat16()
    q, k, v = mk(5000 + s), mk(5001 + s), mk(5002 + s)
    out, lse = D.swa_forward_lse(q, k, v, nh, hd, w, n_p)
    torch.cuda.synchronize()
    assert D.ffi.lib().nlh_swa_tc_timeout_flag() == 0
    for bi in range(b):
        f = orc.swa_forward(_np(q[bi]), _np(k[bi]), _np(v[bi]), nh, hd, w, n_p)
        assert rel_err(_np(out[bi]), f["out"]) <= 2e-2, rel_err(_np(out[bi]), f["out"])
    # same log-sum-exp as the mma.sync kernel (both fp32 accumulate over bf16 products)
    D.call("nlh_set_option", option=1, value=0)
    out2, lse2 = D.swa_forward_lse(q, k, v, nh, hd, w, n_p)
    D.call("nlh_set_option", option=1, value=1)
    assert max_abs(_np(lse), _np(lse2)) < 1e-3
    assert max_abs(_np(out), _np(out2)) < 2e-2
