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


@pytest.mark.parametrize("rule,key", [("delta", "DeltaRule"), ("titans", "TitansLMM"), ("hebbian", "HebbianRule")])
@pytest.mark.parametrize("d,s,pad", [(64, 40, 0), (32, 17, 0), (16, 9, 5), (128, 12, 0)])
def test_rule_level_adapters(D, orc, rule, key, d, s, pad):
    """A whole rule block (projections, L2 norm, gates, inner loop) behind one key: saved buffers in
    the order record_on_tape stores them, d_embedded and the flat parameter gradient out
    (core/src/opaque_adapters.rs:306-628), against the rule-level oracle."""
    from oracle import rule_level as RL
    flat = RL.make_flat(d, 7000 + d + s)
    flat = np.concatenate([flat, np.zeros(pad, np.float32)])          # trailing optional fields
    emb = orc.rand_buf(s * d, 7100 + d, 1.0).reshape(s, d)
    d_y = orc.rand_buf(s * d, 7200 + d, 1.0).reshape(s, d)
    y, saved = RL.record(rule, flat, emb)
    want_emb, want_flat = RL.opaque_backward(rule, d_y, saved, flat.size)
    got_emb, got_flat = D.opaque_backward(key, [d_y], saved, [s * d, flat.size])
    assert rel_err(got_emb, want_emb) <= 1e-4, rel_err(got_emb, want_emb)
    n = RL.flat_len(d)
    parts = RL.split_flat(want_flat, d)
    got_parts = RL.split_flat(got_flat, d)
    for name in parts:
        if np.abs(parts[name]).max() == 0.0:
            assert np.abs(got_parts[name]).max() == 0.0, name          # fields the rule does not have
        else:
            assert rel_err(got_parts[name], parts[name]) <= 1e-4, (name, rel_err(got_parts[name], parts[name]))
    assert np.all(got_flat[n:] == 0.0)


def test_rule_level_adapter_rejects_what_is_off_the_path(D, orc):
    from oracle import rule_level as RL
    d, s = 16, 6
    flat = RL.make_flat(d, 7300)
    emb = orc.rand_buf(s * d, 7301, 1.0).reshape(s, d)
    y, saved = RL.record("titans", flat, emb)
    for idx, val in ((7, 1.0), (12, 2.0), (2, 1.0), (15, 4.0)):     # feature map, MLP memory, L1 bias, conv1d
        bad = [a.copy() for a in saved]
        bad[0][idx] = val
        with pytest.raises(RuntimeError, match="on the path"):
            D.opaque_backward("TitansLMM", [emb], bad, [s * d, flat.size])


def test_unsupported_keys_and_bad_lengths_are_rejected(D):
    meta = np.array([4, 8], dtype=np.float32)
    z = np.zeros(32, dtype=np.float32)
    with pytest.raises(RuntimeError):        # a key off the path: no GPU form
        D.opaque_backward(3, [z], [meta, z], [32])       # OpaqueKey::Moneta
    with pytest.raises(RuntimeError):        # rule-level adapter with too few saved buffers
        D.opaque_backward("TitansLMM", [z], [meta, z], [32])
    with pytest.raises(RuntimeError):        # d_y length does not match meta
        D.opaque_backward("FrozenDeltaRule", [z[:5]], [meta, np.zeros(64, np.float32)], [32])
    with pytest.raises(RuntimeError):        # a feature map other than identity
        D.opaque_backward("FrozenDeltaRule", [z], [np.array([4, 8, 1, 0.5], np.float32), np.zeros(64, np.float32)], [32])
