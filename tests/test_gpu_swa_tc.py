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


@pytest.mark.parametrize("b,s,nh,w,n_p,packed", [(2, 300, 2, 96, 0, False), (1, 513, 2, 512, 0, False),
                                                 (1, 200, 1, 40, 7, False), (3, 512, 4, 512, 0, True),
                                                 (1, 1, 1, 1, 0, False), (2, 1000, 1, 256, 0, True)])
def test_tma_staged_forward_is_used_and_equals_cp_async_staging(tc_on, orc, b, s, nh, w, n_p, packed):
    """NLH_OPT_SWA_TMA: the tcgen05 forward stages Q, K and V with tiled TMA copies (the library
    reports which staging a launch used). Same MMAs on the same operands: the result must equal
    the cp.async staging bit for bit, ragged last tiles (zero-filled out-of-bounds rows), several
    batch elements and the packed q|k|v row layout included."""
    import torch
    D = tc_on
    hd = 64
    d = nh * hd
    g = torch.Generator().manual_seed(50 + s)
    res = {}
    if packed:
        qkv = (torch.randn(b, s, 3 * d, generator=g) * 0.5).cuda().bfloat16()
    else:
        q, k, v = ((torch.randn(b, s, d, generator=g) * 0.5).cuda().bfloat16() for _ in range(3))
    try:
        for tma in (1, 0):
            D.call("nlh_set_option", option=4, value=tma)
            if packed:
                out = torch.empty(b, s, d, dtype=torch.bfloat16, device="cuda")
                lse = torch.empty(b, nh, s, dtype=torch.float32, device="cuda")
                D.call("nlh_swa_forward_packed", qkv=qkv, out=out, lse=lse, seq_len=s, num_heads=nh,
                       head_dim=hd, window_size=w, batch_size=b, n_persistent=n_p)
            else:
                out, lse = D.swa_forward_lse(q, k, v, nh, hd, w, n_p)
            torch.cuda.synchronize()
            assert D.ffi.lib().nlh_swa_forward_staging() == tma
            assert D.ffi.lib().nlh_swa_tc_timeout_flag() == 0
            res[tma] = (out.clone(), lse.clone())
    finally:
        D.call("nlh_set_option", option=4, value=1)
    assert torch.equal(res[1][0], res[0][0]) and torch.equal(res[1][1], res[0][1])
    if not packed:
        for bi in range(b):
            f = orc.swa_forward(_np(q[bi]), _np(k[bi]), _np(v[bi]), nh, hd, w, n_p)
            assert rel_err(_np(res[1][0][bi]), f["out"]) <= 2e-2
