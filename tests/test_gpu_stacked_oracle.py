"""GPU: the stacked model on this library's kernels against the stacked-model oracle
(oracle/stacked.py: restatement of core/src/traced_forward.rs:1313-1499 with the GPU-resident
level semantics, forward and backward) — identical seeded initialisation, identical token ids,
loss and EVERY parameter gradient, over two consecutive calls (the second one starts from carried
memories). k = 4 CMS levels with the cfg3 chunk sizes [1, 8, 64, 512] (clipped to the sequence).
The configuration runs in fp32 (fp32 SWA pair, fp32 GEMMs), so it is held to the fp32 bar of
1e-4 relative (per tensor: max |got - want| / max |want|)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4


def _cfgs(**kw):
    from nl_hecate_b200.stacked_mag import StackedMAGConfig
    from oracle import stacked as ST
    base = dict(d_model=128, num_heads=2, n_blocks=2, k=4, chunk_sizes=(1, 8, 64, 512), seq_len=64,
                window=32, vocab=512, exact_levels=(0,))
    base.update(kw)
    gcfg = StackedMAGConfig(bf16=False, tie_embeddings=False, level_streams=False, **base)
    ocfg = ST.Cfg(mode="resident", **base)
    return gcfg, ocfg


def test_seeded_init_is_the_reference_init_bit_for_bit(orc):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import StackedMAG
    from oracle import stacked as ST
    gcfg, ocfg = _cfgs()
    m = StackedMAG(gcfg, batch_per_rank=1, seed=42)
    p = ST.init_params(ocfg, seed=42)
    assert set(p) == set(m.p)
    for n, a in p.items():
        assert np.array_equal(m.p[n].detach().cpu().numpy(), a.reshape(m.p[n].shape)), n


@pytest.mark.parametrize("stream", [False, True])
@pytest.mark.parametrize("kw", [dict(), dict(d_model=64, num_heads=1, k=2, chunk_sizes=(1, 1), exact_levels=(0, 1))])
def test_stacked_model_matches_the_stacked_oracle(orc, kw, stream, monkeypatch):
    """stream: the pooled levels with short chunks run the full-trajectory frozen pair (what the
    model picks at large problem counts) or the chunk-boundary pair (small problem counts)."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import stacked_mag
    from nl_hecate_b200.stacked_mag import StackedMAG
    from oracle import stacked as ST
    monkeypatch.setattr(stacked_mag._TitansMemory, "STREAM_MIN_PROBLEMS", 0 if stream else 10 ** 9)
    gcfg, ocfg = _cfgs(**kw)
    B, S = 2, gcfg.seq_len
    m = StackedMAG(gcfg, batch_per_rank=B, seed=42)
    p = ST.init_params(ocfg, seed=42)
    rng = np.random.default_rng(3)
    for n in p:                                   # make every branch matter
        base = n.split(".")[-1]
        if base.endswith("gamma"):
            p[n] = (p[n] + 0.2 * rng.standard_normal(p[n].shape)).astype(np.float32)
        elif base.endswith("beta") or base == "alpha_mem":
            p[n] = (p[n] + 0.3 * rng.standard_normal(p[n].shape)).astype(np.float32)
        elif base == "b_theta":
            p[n] = np.array([-2.0], np.float32)
        elif base == "b_alpha":
            p[n] = np.array([-1.0], np.float32)
        elif base == "w_kvq_mem":
            p[n] = (p[n] * 2.0).astype(np.float32)
    with torch.no_grad():
        for n, a in p.items():
            m.p[n].copy_(torch.from_numpy(a).view(m.p[n].shape))
    ids = orc.rng_tokens(7, gcfg.vocab, 2 * B * (S + 1)).reshape(2, B, S + 1)
    ctxs = [ST.new_context(ocfg) for _ in range(B)]
    worst = {}
    for call in range(2):
        x, t = ids[call, :, :-1], ids[call, :, 1:]
        losses, grads = [], None
        for b in range(B):
            l, g = ST.forward_backward(p, x[b], t[b], ctxs[b], ocfg)
            losses.append(l)
            grads = g if grads is None else {k_: grads[k_] + g[k_] for k_ in g}
        want_loss = float(np.mean(losses))
        m.opt.g.zero_()
        got_loss = float(m.forward_backward(torch.from_numpy(np.ascontiguousarray(x)).cuda().long(),
                                            torch.from_numpy(np.ascontiguousarray(t)).cuda().long()))
        assert abs(got_loss - want_loss) <= TOL * abs(want_loss), (call, got_loss, want_loss)
        for n, w in grads.items():
            w = w / B
            a = m.g[n].detach().cpu().numpy().reshape(w.shape)
            e = float(np.abs(a - w).max() / max(np.abs(w).max(), 1e-12))
            worst[n.split(".")[-1]] = max(worst.get(n.split(".")[-1], 0.0), e)
            assert e <= TOL, (call, n, e)
        # carried memories agree as well
        for bl in range(gcfg.n_blocks):
            for l in range(gcfg.k):
                got = m.context[bl][l].detach().cpu().numpy()
                want = np.concatenate([ctxs[b][bl][l] for b in range(B)], axis=0)
                assert np.abs(got - want).max() <= TOL * max(np.abs(want).max(), 1e-9), (call, bl, l)
    print("stacked model vs oracle, worst relative gradient errors per tensor kind:", worst)
