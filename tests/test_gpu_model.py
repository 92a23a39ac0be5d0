"""GPU: the stacked MAG harness with this library's kernels vs the same harness with the
plain-PyTorch statements of the operators (tests/torch_ref.py), on a small configuration.
SWA runs in bf16 on tensor cores, so gradients are compared at the bf16 bar (2e-2 relative,
against the largest entry of the tensor); the loss at 1e-3."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from torch_ref import swa_ref, titans_memory_ref  # noqa: E402

pytestmark = pytest.mark.gpu


def _cfg(bf16, fused=True):
    from nl_hecate_b200.stacked_mag import StackedMAGConfig
    return StackedMAGConfig(d_model=128, num_heads=2, n_blocks=2, k=3, chunk_sizes=(1, 4, 16),
                            seq_len=32, window=16, vocab=96, bf16=bf16, fused_glue=fused)


def _data(batch, seed=0):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, 96, (batch, 33), generator=g)
    return tok[:, :-1].contiguous().cuda(), tok[:, 1:].contiguous().cuda()


def _compare(ours, ref, tok, tgt, loss_tol, grad_tol, l2=False):
    for _ in range(2):     # second pass runs with non-zero carried memories
        ours.opt.g.zero_(); ref.opt.g.zero_()
        lo = ours.forward_backward(tok, tgt)
        lr = ref.forward_backward(tok, tgt)
        assert abs(float(lo) - float(lr)) <= loss_tol * abs(float(lr)), (float(lo), float(lr))
    worst = ("", 0.0)
    for i, n in enumerate(ours.names):
        a, b = ours.opt.view(ours.opt.g, i), ref.opt.view(ref.opt.g, i)
        denom = float(b.abs().max())
        if denom < 1e-7:
            assert float(a.abs().max()) < 1e-5, n
            continue
        if l2:
            if a.numel() < 64:
                continue   # scalar gate biases: cancelling sums, dominated by bf16 noise
            err = float((a - b).norm() / b.norm())
        else:
            err = float((a - b).abs().max()) / denom
        if err > worst[1]:
            worst = (n, err)
    assert worst[1] <= grad_tol, worst
    for b in range(2):
        for l in range(3):
            a, r = ours.context[b][l], ref.context[b][l]
            assert float((a - r).abs().max()) <= max(grad_tol, 1e-3) * max(float(r.abs().max()), 1e-6)


def test_memory_kernels_inside_the_model_match_torch_reference():
    """fp32 path: this library's memory kernels + the torch SWA statement vs all-torch.
    Every parameter gradient within 2e-3 of the tensor's largest entry (different summation
    orders through two blocks and three CMS levels), loss within 1e-5."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import StackedMAG
    tok, tgt = _data(3)
    ours = StackedMAG(_cfg(False), 3, device="cuda", seed=1, swa_fn=swa_ref)
    ref = StackedMAG(_cfg(False, fused=False), 3, device="cuda", seed=1, memory_fn=titans_memory_ref,
                     swa_fn=swa_ref)
    assert torch.equal(ours.opt.w, ref.opt.w)
    _compare(ours, ref, tok, tgt, 1e-5, 2e-3)


@pytest.mark.parametrize("bf16", [False, True])
def test_full_kernel_path_matches_torch_reference_at_bf16_bar(bf16):
    """All kernels (bf16 tensor-core SWA included) vs all-torch: loss within 1e-3; every
    gradient tensor within 5e-2 in relative L2 norm (scalar gate biases are skipped: they are
    cancelling sums in which the bf16 rounding of the attention probabilities dominates)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import StackedMAG
    tok, tgt = _data(3)
    ours = StackedMAG(_cfg(bf16), 3, device="cuda", seed=1)
    ref = StackedMAG(_cfg(bf16, fused=False), 3, device="cuda", seed=1, memory_fn=titans_memory_ref,
                     swa_fn=swa_ref)
    _compare(ours, ref, tok, tgt, 1e-3, 5e-2, l2=True)


def test_training_steps_reduce_loss_and_tie_embeddings():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import StackedMAG
    m = StackedMAG(_cfg(True), 4, device="cuda", seed=3)
    m.cfg.lr = 3e-3
    tok, tgt = _data(4, seed=5)
    losses = [float(m.step(tok, tgt)) for _ in range(8)]
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] < losses[0] - 0.05, losses
    assert torch.equal(m.p["w_embed"], m.p["w_unembed"].t())
    assert m.global_step == 8 and m.level_steps == [8, 8, 8]
    assert float(m.opt.g.abs().max()) == 0.0     # gradient arena cleared for the next step
    # b_theta stays inside its clamp
    for n, w in m.p.items():
        if n.endswith("b_theta"):
            assert -10.0 <= float(w.detach()) <= 2.0


@pytest.mark.parametrize("bf16", [False, True])
def test_fused_glue_matches_torch_glue(bf16):
    """Same kernels for memory and SWA in both models; only the rule wrapper / MAG combine differ
    (fused CUDA kernels vs PyTorch ops). fp32: gradients within 1e-3 of each tensor's largest
    entry; bf16: within 3e-2 in relative L2 norm (the fused path rounds d_kvq to bf16 once)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import StackedMAG
    tok, tgt = _data(3)
    fused = StackedMAG(_cfg(bf16, True), 3, device="cuda", seed=2)
    plain = StackedMAG(_cfg(bf16, False), 3, device="cuda", seed=2)
    if bf16:
        _compare(fused, plain, tok, tgt, 1e-3, 3e-2, l2=True)
    else:
        _compare(fused, plain, tok, tgt, 1e-5, 1e-3)


def test_graph_replayed_step_matches_eager_steps():
    """step_graphed = 2 eager steps + capture + replay on the first call, replay afterwards: after
    the same number of steps the parameters agree with a model stepped eagerly."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import StackedMAG
    tok, tgt = _data(4, seed=9)
    eager = StackedMAG(_cfg(True), 4, device="cuda", seed=7)
    graph = StackedMAG(_cfg(True), 4, device="cuda", seed=7)
    for _ in range(5):
        le = eager.step(tok, tgt)
    lg = graph.step_graphed(tok, tgt)        # steps 1-3
    for _ in range(2):
        lg = graph.step_graphed(tok, tgt)    # steps 4, 5
    torch.cuda.synchronize()
    assert graph.global_step == eager.global_step == 5
    assert abs(float(le) - float(lg)) <= 1e-3 * abs(float(le))
    err = float((eager.opt.w - graph.opt.w).abs().max())
    assert err <= 1e-4, err
    for b in range(2):
        for l in range(3):
            a, r = graph.context[b][l], eager.context[b][l]
            assert float((a - r).abs().max()) <= 1e-3 * max(float(r.abs().max()), 1e-6)


def test_checkpointed_exact_level_matches_the_stored_trajectory():
    """cfg.exact_checkpoint: level 0 keeps a checkpoint every 8 tokens and recomputes the windows in
    the backward: same loss and gradients as the stored-trajectory pair (both fp32 state; the
    stored-M pair derives S from M differences, so agreement is to fp32 rounding)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import dataclasses
    from nl_hecate_b200.stacked_mag import StackedMAG
    tok, tgt = _data(3, seed=4)
    full = StackedMAG(_cfg(True), 3, device="cuda", seed=5)
    ckpt = StackedMAG(dataclasses.replace(_cfg(True), exact_checkpoint=8), 3, device="cuda", seed=5)
    for _ in range(2):
        full.opt.g.zero_(); ckpt.opt.g.zero_()
        lf = full.forward_backward(tok, tgt)
        lc = ckpt.forward_backward(tok, tgt)
    assert abs(float(lf) - float(lc)) <= 1e-6 * abs(float(lf))
    for i, n in enumerate(full.names):
        a, b = ckpt.opt.view(ckpt.opt.g, i), full.opt.view(full.opt.g, i)
        denom = max(float(b.abs().max()), 1e-7)
        assert float((a - b).abs().max()) <= 2e-4 * denom, n


def test_level_streams_match_single_stream_eager_and_graphed():
    """cfg.level_streams issues CMS levels >= 1 on side streams (own scratch slots): the same
    kernels run, so gradients agree with the single-stream model to rounding (only the order of
    the atomic adds into shared gradients can differ), eagerly and replayed from the graph."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import dataclasses
    from nl_hecate_b200.stacked_mag import StackedMAG
    tok, tgt = _data(4, seed=21)
    cfg_s = dataclasses.replace(_cfg(True), level_streams=True)
    cfg_1 = dataclasses.replace(_cfg(True), level_streams=False)
    multi = StackedMAG(cfg_s, 4, device="cuda", seed=5)
    single = StackedMAG(cfg_1, 4, device="cuda", seed=5)
    _compare(multi, single, tok, tgt, 1e-6, 1e-4)
    multi = StackedMAG(cfg_s, 4, device="cuda", seed=6)
    single = StackedMAG(cfg_1, 4, device="cuda", seed=6)
    for _ in range(5):
        le = single.step(tok, tgt)
    for _ in range(3):
        lg = multi.step_graphed(tok, tgt)     # steps 1-3 on the first call, then 4 and 5
    torch.cuda.synchronize()
    assert multi.global_step == single.global_step == 5
    assert abs(float(le) - float(lg)) <= 1e-3 * abs(float(le))
    assert float((single.opt.w - multi.opt.w).abs().max()) <= 1e-4
