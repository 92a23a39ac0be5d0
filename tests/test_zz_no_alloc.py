"""GPU test of nlh_titans_backward_noalloc, the backward entry for hosts that cannot let the
library allocate device memory (their own pool owns the device, or an allocation's implicit
device synchronisation is not acceptable where they call from).

The entry keeps its scratch in a fixed array inside the library, so it must (a) agree with
the allocating entry titans_backward_f32_cuda, (b) give the right answer on a second call that
finds the first call's leftovers in the shared array, (c) refuse sizes beyond its limit and
NULL buffers (it has no M-only mode), and (d) leave the device's free memory and the library's
own workspace exactly as it found them. The test does not depend on anything other tests leave
behind.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL = 1e-4


def _rel(got, want):
    got = got.detach().cpu().numpy().astype(np.float64)
    want = want.detach().cpu().numpy().astype(np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-12))


def _problem(torch, n, s, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *sh: (torch.rand(*sh, generator=g, device="cuda") * 2 - 1)
    k, v, q, dy = (0.1 * r(n, s, d) for _ in range(4))
    alpha, theta, eta = (0.5 + 0.4 * r(n, s) for _ in range(3))
    m0, s0 = 0.1 * r(n, d * d), 0.1 * r(n, d * d)
    return k, v, q, alpha, theta, eta, m0, s0, dy


def _noalloc_backward(D, torch, k, v, q, alpha, theta, eta, ms, ss, dy):
    n, s, d = k.shape
    dk, dv, dq = (torch.full_like(k, float("nan")) for _ in range(3))
    da, dt, de = (torch.full_like(alpha, float("nan")) for _ in range(3))
    dm0 = torch.zeros(d * d, device="cuda")
    ds0 = torch.zeros(d * d, device="cuda")
    D.call("nlh_titans_backward_noalloc", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
           eta=eta, m_states=ms, s_states=ss, d_y=dy, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq,
           d_alpha=da, d_theta=dt, d_eta=de, d_m_initial=dm0, d_s_initial=ds0, seq_len=s, d=d,
           batch_size=n, error_clip=0.0)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dt, d_eta=de, d_m_initial=dm0,
                d_s_initial=ds0)


def test_noalloc_backward_matches_allocating_entry_twice():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch as D
    # two calls in a row with different shapes and data: the second one runs on top of
    # whatever the first left in the shared array
    # d = 128 runs the several-row-groups branch of the kernel, d = 512 its column loop
    for n, s, d, seed in ((3, 20, 64, 11), (5, 9, 32, 12), (2, 6, 128, 13), (1, 3, 512, 14)):
        k, v, q, alpha, theta, eta, m0, s0, dy = _problem(torch, n, s, d, seed)
        ms, ss, _ = D.titans_forward_dd(k, v, q, alpha, theta, eta, m0, s0)
        want = D.titans_backward_dd(k, v, q, alpha, theta, eta, ms, ss, dy)
        got = _noalloc_backward(D, torch, k, v, q, alpha, theta, eta, ms, ss, dy)
        torch.cuda.synchronize()
        for key in want:
            assert torch.isfinite(got[key]).all(), key
            assert _rel(got[key], want[key]) <= REL, (n, s, d, key, _rel(got[key], want[key]))


def test_noalloc_backward_rejects_sizes_beyond_the_builtin_scratch():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch as D
    z = torch.zeros(8, device="cuda")
    # 65 problems at d = 64 need 266240 floats per accumulator > 262144
    with pytest.raises(RuntimeError, match="exceeds the built-in scratch"):
        D.call("nlh_titans_backward_noalloc", k_mem=z, v_mem=z, q_mem=z, alpha=z, theta=z, eta=z,
               m_states=z, s_states=z, d_y=z, d_k_mem=z, d_v_mem=z, d_q_mem=z, d_alpha=z,
               d_theta=z, d_eta=z, d_m_initial=z, d_s_initial=z, seq_len=4, d=64, batch_size=65,
               error_clip=0.0)


def test_noalloc_backward_allocates_nothing():
    """After one warm-up call (which looks up the array's device address), a call must leave the
    device's free memory and the library's workspace size unchanged."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch as D
    k, v, q, alpha, theta, eta, m0, s0, dy = _problem(torch, 4, 12, 64, 21)
    ms, ss, _ = D.titans_forward_dd(k, v, q, alpha, theta, eta, m0, s0)
    _noalloc_backward(D, torch, k, v, q, alpha, theta, eta, ms, ss, dy)       # warm-up / set-up
    # outputs allocated up front so that torch's own allocator is quiet during the checked call
    n, s, d = k.shape
    outs = dict(d_k_mem=torch.empty_like(k), d_v_mem=torch.empty_like(k), d_q_mem=torch.empty_like(k),
                d_alpha=torch.empty_like(alpha), d_theta=torch.empty_like(alpha),
                d_eta=torch.empty_like(alpha), d_m_initial=torch.zeros(d * d, device="cuda"),
                d_s_initial=torch.zeros(d * d, device="cuda"))
    torch.cuda.synchronize()
    lib = D.ffi.lib()
    ws_before = int(lib.nlh_workspace_bytes())
    free_before, _ = torch.cuda.mem_get_info()
    D.call("nlh_titans_backward_noalloc", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
           eta=eta, m_states=ms, s_states=ss, d_y=dy, seq_len=s, d=d, batch_size=n, error_clip=0.0,
           **outs)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert int(lib.nlh_workspace_bytes()) == ws_before
    assert free_after == free_before
    assert torch.isfinite(outs["d_k_mem"]).all()


def test_noalloc_backward_rejects_null_buffers_on_the_host():
    """The entry has no M-only mode: s_states = NULL (valid for titans_backward_f32_cuda) and any
    other missing buffer are refused before anything is launched."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch as D
    z = torch.zeros(64, device="cuda")
    base = dict(k_mem=z, v_mem=z, q_mem=z, alpha=z, theta=z, eta=z, m_states=z, s_states=z, d_y=z,
                d_k_mem=z, d_v_mem=z, d_q_mem=z, d_alpha=z, d_theta=z, d_eta=z, d_m_initial=z,
                d_s_initial=z, seq_len=1, d=4, batch_size=1, error_clip=0.0)
    for missing in ("s_states", "theta", "d_eta"):
        kw = dict(base)
        kw[missing] = None
        with pytest.raises(RuntimeError, match="NULL pointer"):
            D.call("nlh_titans_backward_noalloc", **kw)
