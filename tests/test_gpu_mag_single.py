"""GPU: the reference's CPU-runnable configuration — single-block MAG, one memory level, Delta
rule, d_model 64, one head of 64, seq 256, window 256, vocab 256, batch 2 — on this library's
kernels (nl_hecate_b200/mag_single.py) against the model-level oracle (oracle/mag_single.py, a
restatement of core/src/mag.rs mag_forward / mag_backward): the loss and EVERY parameter
gradient. The configuration is fp32, so it runs fp32 end to end (fp32 SWA pair) and is held to the
fp32 bar: loss and every gradient within 1e-4 relative (of each tensor's largest entry), gate
biases included. The same model with the attention branch on the bf16 tensor-core pair is held to
the bf16 bar, 2e-2 on every tensor. A Titans variant on a smaller shape covers the second rule
wrapper."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(orc, rule, d, nh, s, vocab, window, batch, seed, fp32_swa=True):
    import torch
    from oracle import mag_single as O
    from nl_hecate_b200.mag_single import MAGSingle
    p = O.init_params(d, vocab, seed=seed, rule=rule)
    for n in ("w_k_mem", "w_v_mem", "w_q_mem"):            # a memory branch that matters
        p[n] = (p[n] * 2.0).astype(np.float32)
    ids = orc.rng_tokens(7, vocab, batch * (s + 1)).reshape(batch, s + 1)
    x, t = ids[:, :-1], ids[:, 1:]
    losses, grads = [], None
    for b in range(batch):
        l, g = O.forward_backward(p, x[b], t[b], nh, window, rule)
        losses.append(l)
        grads = g if grads is None else {k: grads[k] + g[k] for k in g}
    want_loss = float(np.mean(losses))
    want = {k: v / batch for k, v in grads.items()}
    model = MAGSingle(p, nh, window, rule, fp32_swa=fp32_swa)
    got_loss, got = model.loss_and_grads(torch.from_numpy(np.ascontiguousarray(x)).cuda().long(),
                                         torch.from_numpy(np.ascontiguousarray(t)).cuda().long())
    tol = 1e-4 if fp32_swa else 2e-2
    assert abs(got_loss - want_loss) <= (1e-4 if fp32_swa else 2e-3) * abs(want_loss), (got_loss, want_loss)
    assert set(got) == set(want), sorted(set(want) ^ set(got))
    errs = {}
    for name, w in want.items():
        a = got[name].float().cpu().numpy().reshape(w.shape)
        denom = max(float(np.abs(w).max()), 1e-12)
        errs[name] = (round(float(np.abs(a - w).max()) / denom, 5), float(np.abs(w).max()))
    bad = {n: e for n, e in errs.items() if e[0] > tol}
    assert not bad, (bad, errs)
    print(f"{rule} fp32_swa={fp32_swa}: loss rel err {abs(got_loss - want_loss) / abs(want_loss):.2e}, "
          f"worst gradient rel err {max(e[0] for e in errs.values()):.2e}")


def test_cfg1_delta_mag_matches_the_model_oracle(orc):
    if not __import__("torch").cuda.is_available():
        pytest.skip("needs a CUDA device")
    _run(orc, "delta", d=64, nh=1, s=256, vocab=256, window=256, batch=2, seed=42)


def test_cfg1_with_bf16_attention_meets_the_bf16_bar(orc):
    if not __import__("torch").cuda.is_available():
        pytest.skip("needs a CUDA device")
    _run(orc, "delta", d=64, nh=1, s=256, vocab=256, window=256, batch=2, seed=42, fp32_swa=False)


def test_titans_mag_single_matches_the_model_oracle(orc):
    if not __import__("torch").cuda.is_available():
        pytest.skip("needs a CUDA device")
    _run(orc, "titans", d=64, nh=2, s=96, vocab=128, window=32, batch=2, seed=43)
