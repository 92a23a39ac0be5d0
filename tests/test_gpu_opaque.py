"""GPU: the C-ABI opaque-VJP entry (host slices in, host slices out) vs the CPU oracle, with the
saved-buffer layouts of core/src/opaque_adapters.rs. fp32 adapters at relative 1e-4; the SWA
adapter rounds q,k,v to bf16 on the device (2e-2 against the oracle fed the rounded inputs)."""
import numpy as np
import pytest

from helpers import make_problem, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def D():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch
    return dispatch


@pytest.mark.parametrize("d,s", [(64, 24), (16, 9)])
def test_dgd_adapter(D, orc, d, s):
    p = make_problem(orc, 1, s, d, 3100 + d, "rand")
    f = orc.delta_forward(p["k"][0], p["v"][0], p["q"][0], p["alpha"][0], p["theta"][0], p["m0"][0])
    want = orc.delta_backward(p["k"][0], p["v"][0], p["q"][0], p["alpha"][0], p["theta"][0],
                              f["m_states"], p["dy"][0])
    meta = np.array([s, d], dtype=np.float32)
    saved = [meta, p["k"][0], p["v"][0], p["q"][0], p["alpha"][0], p["theta"][0], f["m_states"]]
    got = D.opaque_backward("DGD", [p["dy"][0]], saved, [s * d, s * d, s * d, s, s, d * d])
    for g, key in zip(got, ("d_k", "d_v", "d_q", "d_alpha", "d_theta", "d_m_initial")):
        assert rel_err(g, np.asarray(want[key]).ravel()) <= 1e-4, key


def test_swa_adapter(D, orc):
    s, nh, hd, w = 96, 2, 32, 24
    n = s * nh * hd
    q, k, v = (orc.bf16_round(orc.rand_buf(n, 3200 + i, 0.5)) for i in range(3))
    d_out = orc.rand_buf(n, 3203, 1.0)
    shape = (s, nh * hd)
    f = orc.swa_forward(q.reshape(shape), k.reshape(shape), v.reshape(shape), nh, hd, w)
    want = orc.swa_backward(q.reshape(shape), k.reshape(shape), v.reshape(shape), f["attn_weights"],
                            d_out.reshape(shape), nh, hd, w)
    meta = np.array([s, nh, hd, w], dtype=np.float32)
    got = D.opaque_backward("SWA", [d_out], [meta, q, k, v, f["attn_weights"]], [n, n, n])
    for g, key in zip(got, ("d_q", "d_k", "d_v")):
        assert rel_err(g, np.asarray(want[key]).ravel()) <= 2e-2, key


@pytest.mark.parametrize("key", ["FrozenDeltaRule", "FrozenTitansLMM", "FrozenHebbianRule"])
def test_frozen_read_adapter(D, orc, key):
    s, d = 13, 32
    m = orc.rand_buf(d * d, 3300, 1.0).reshape(d, d)
    dy = orc.rand_buf(s * d, 3301, 1.0).reshape(s, d)
    got = D.opaque_backward(key, [dy], [np.array([s, d], dtype=np.float32), m], [s * d])[0]
    want = (dy.astype(np.float64) @ m.astype(np.float64)).ravel()     # d_q[t] = M^T d_y[t]
    assert rel_err(got, want) <= 1e-5


def test_unsupported_keys_and_bad_lengths_are_rejected(D):
    meta = np.array([4, 8], dtype=np.float32)
    z = np.zeros(32, dtype=np.float32)
    with pytest.raises(RuntimeError):        # rule-level adapter: no GPU form
        D.opaque_backward("TitansLMM", [z], [meta, z], [32])
    with pytest.raises(RuntimeError):        # d_y length does not match meta
        D.opaque_backward("FrozenDeltaRule", [z[:5]], [meta, np.zeros(64, np.float32)], [32])
    with pytest.raises(RuntimeError):        # a feature map other than identity
        D.opaque_backward("FrozenDeltaRule", [z], [np.array([4, 8, 1, 0.5], np.float32), np.zeros(64, np.float32)], [32])
