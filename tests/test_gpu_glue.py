"""GPU: LayerNorm, cross-entropy and embedding kernels vs the CPU oracle, through the C ABI.
fp32 entries: abs error <= 2e-5 (forward) / 1e-4 relative (reductions over thousands of rows);
bf16 variants: 1e-2 relative (bf16 rounding of the stored values)."""
import numpy as np
import pytest

from helpers import max_abs, rel_err

pytestmark = pytest.mark.gpu


def _dev(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def _np(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("n,d", [(1, 4), (37, 512), (300, 50), (65, 1024), (9, 1536), (2048, 128)])
def test_layer_norm_drop_in_matches_oracle(orc, n, d):
    import torch
    from nl_hecate_b200 import dispatch as D
    x = orc.rand_buf(n * d, 700 + d, 2.0).reshape(n, d)
    gamma = 1.0 + orc.rand_buf(d, 701, 0.3)
    beta = orc.rand_buf(d, 702, 0.2)
    dy = orc.rand_buf(n * d, 703, 1.0).reshape(n, d)
    out_r, mean_r, rstd_r = orc.layer_norm_forward(x, gamma, beta, 1e-5)
    dx_r, dg_r, db_r = orc.layer_norm_backward(dy, x, gamma, mean_r, rstd_r)
    xd, gd, bd, dyd = _dev(x), _dev(gamma), _dev(beta), _dev(dy)
    out, mean, rstd = torch.empty_like(xd), torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
    D.call("layer_norm_forward_cuda", x=xd, gamma=gd, beta=bd, out=out, mean_cache=mean,
           rstd_cache=rstd, n=n, d=d, eps=1e-5)
    assert max_abs(_np(out), out_r) <= 2e-5
    assert max_abs(_np(mean), mean_r) <= 1e-6 and rel_err(_np(rstd), rstd_r) <= 1e-5
    dx = torch.empty_like(xd)
    dgb = torch.zeros(2, d, device="cuda")
    D.call("layer_norm_backward_cuda", d_out=dyd, x=xd, gamma=gd, mean_cache=mean, rstd_cache=rstd,
           d_x=dx, d_gamma=dgb[0], d_beta=dgb[1], n=n, d=d)
    assert rel_err(_np(dx), dx_r) <= 1e-4
    assert rel_err(_np(dgb[0]), dg_r) <= 1e-4 and rel_err(_np(dgb[1]), db_r) <= 1e-4
    # the backward accumulates into the parameter gradients
    D.call("layer_norm_backward_cuda", d_out=dyd, x=xd, gamma=gd, mean_cache=mean, rstd_cache=rstd,
           d_x=dx, d_gamma=dgb[0], d_beta=dgb[1], n=n, d=d)
    assert rel_err(_np(dgb[0]), 2 * dg_r) <= 1e-4


def test_layer_norm_bf16_outputs_and_split_gradient(orc):
    import torch
    from nl_hecate_b200 import dispatch as D
    n, d = 129, 512
    x = orc.rand_buf(n * d, 711, 2.0).reshape(n, d)
    gamma = 1.0 + orc.rand_buf(d, 712, 0.3)
    beta = orc.rand_buf(d, 713, 0.2)
    g32 = orc.rand_buf(n * d, 714, 1.0).reshape(n, d)
    g16 = orc.bf16_round(orc.rand_buf(n * d, 715, 1.0).reshape(n, d))
    out_r, mean_r, rstd_r = orc.layer_norm_forward(x, gamma, beta, 1e-5)
    dx_r, dg_r, db_r = orc.layer_norm_backward(g32 + g16, x, gamma, mean_r, rstd_r)
    xd, gd, bd = _dev(x), _dev(gamma), _dev(beta)
    o32 = torch.empty_like(xd)
    o16 = torch.empty(n, d, dtype=torch.bfloat16, device="cuda")
    mean, rstd = torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
    D.call("nlh_layer_norm_forward", x=xd, gamma=gd, beta=bd, out_f32=o32, out_bf16=o16,
           mean_cache=mean, rstd_cache=rstd, n=n, d=d, eps=1e-5)
    assert max_abs(_np(o32), out_r) <= 2e-5
    assert np.array_equal(_np(o16), orc.bf16_round(_np(o32)))
    dx = torch.empty_like(xd)
    dgb = torch.zeros(2, d, device="cuda")
    D.call("nlh_layer_norm_backward", d_out_f32=_dev(g32), d_out_bf16=_dev(g16, torch.bfloat16), x=xd,
           gamma=gd, mean_cache=mean, rstd_cache=rstd, d_x=dx, d_gamma=dgb[0], d_beta=dgb[1], n=n, d=d)
    assert rel_err(_np(dx), dx_r) <= 1e-4
    assert rel_err(_np(dgb[0]), dg_r) <= 1e-4 and rel_err(_np(dgb[1]), db_r) <= 1e-4


@pytest.mark.parametrize("B,S,d,pools,bf16", [(2, 64, 512, (8, 64), True), (3, 48, 128, (2, 8, 24), False),
                                             (1, 512, 512, (8, 64, 512), True), (5, 6, 64, (3,), False)])
def test_layer_norm_backward_with_pooled_sources(orc, B, S, d, pools, bf16):
    """nlh_layer_norm_backward_pooled == oracle LayerNorm backward of (direct gradient + the
    upsampled, 1/c-scaled gradients of the mean-pooled copies); odd row counts exercise the
    two-rows-per-pass tail."""
    import torch
    from nl_hecate_b200 import dispatch as D
    n = B * S
    x = orc.rand_buf(n * d, 721, 2.0).reshape(n, d)
    gamma = 1.0 + orc.rand_buf(d, 722, 0.3)
    beta = orc.rand_buf(d, 723, 0.2)
    g_main = orc.rand_buf(n * d, 724, 1.0).reshape(n, d)
    if bf16:
        g_main = orc.bf16_round(g_main)
    gp = []
    for i, c in enumerate(pools):
        g = orc.rand_buf(B * (S // c) * d, 730 + i, 1.0).reshape(B, S // c, d)
        gp.append(orc.bf16_round(g) if bf16 else g)
    total = g_main.reshape(B, S, d).copy()
    for g, c in zip(gp, pools):
        total += np.repeat(g, c, axis=1) / np.float32(c)
    out_r, mean_r, rstd_r = orc.layer_norm_forward(x, gamma, beta, 1e-5)
    dx_r, dg_r, db_r = orc.layer_norm_backward(total.reshape(n, d), x, gamma, mean_r, rstd_r)
    dt = torch.bfloat16 if bf16 else None
    xd, gd = _dev(x), _dev(gamma)
    mean, rstd = _dev(mean_r), _dev(rstd_r)
    gm = _dev(g_main, dt)
    gpd = [_dev(g, dt) for g in gp] + [None] * (3 - len(gp))
    cs = list(pools) + [1] * (3 - len(pools))
    dx = torch.empty_like(xd)
    dgb = torch.zeros(2, d, device="cuda")
    D.call("nlh_layer_norm_backward_pooled", d_out_f32=None if bf16 else gm, d_out_bf16=gm if bf16 else None,
           g0=gpd[0], c0=cs[0], g0_is_bf16=int(bf16), g1=gpd[1], c1=cs[1], g1_is_bf16=int(bf16),
           g2=gpd[2], c2=cs[2], g2_is_bf16=int(bf16), n_src=len(pools), seq=S, x=xd, gamma=gd,
           mean_cache=mean, rstd_cache=rstd, d_x=dx, d_gamma=dgb[0], d_beta=dgb[1], n=n, d=d)
    assert rel_err(_np(dx), dx_r) <= 1e-4
    assert rel_err(_np(dgb[0]), dg_r) <= 1e-4 and rel_err(_np(dgb[1]), db_r) <= 1e-4
    # pooled sources alone (no direct gradient)
    dx2 = torch.empty_like(xd)
    dgb2 = torch.zeros(2, d, device="cuda")
    D.call("nlh_layer_norm_backward_pooled", d_out_f32=None, d_out_bf16=None,
           g0=gpd[0], c0=cs[0], g0_is_bf16=int(bf16), g1=gpd[1], c1=cs[1], g1_is_bf16=int(bf16),
           g2=gpd[2], c2=cs[2], g2_is_bf16=int(bf16), n_src=len(pools), seq=S, x=xd, gamma=gd,
           mean_cache=mean, rstd_cache=rstd, d_x=dx2, d_gamma=dgb2[0], d_beta=dgb2[1], n=n, d=d)
    dx_r2, _, _ = orc.layer_norm_backward((total - g_main.reshape(B, S, d)).reshape(n, d), x, gamma, mean_r, rstd_r)
    assert rel_err(_np(dx2), dx_r2) <= 1e-4
    # a pool factor that does not divide the sequence is rejected on the host
    with pytest.raises(Exception):
        D.call("nlh_layer_norm_backward_pooled", d_out_f32=None, d_out_bf16=None,
               g0=gpd[0], c0=S + 1, g0_is_bf16=int(bf16), g1=None, c1=1, g1_is_bf16=0, g2=None, c2=1,
               g2_is_bf16=0, n_src=1, seq=S, x=xd, gamma=gd, mean_cache=mean, rstd_cache=rstd, d_x=dx2,
               d_gamma=dgb2[0], d_beta=dgb2[1], n=n, d=d)


@pytest.mark.parametrize("B,S,d,pools", [(2, 64, 512, (8, 64)), (3, 7, 128, ()), (1, 33, 1024, (3,))])
def test_layer_norm_with_residual_operand_and_gradient_fan_in(orc, B, S, d, pools):
    """nlh_layer_norm_residual_forward / nlh_layer_norm_backward_fused: LayerNorm of x + res (bf16
    res), pooled sources, add_in into d_x and the bf16 copy of the input gradient with its own
    addend — against the oracle's LayerNorm on the explicit sum."""
    import torch
    from nl_hecate_b200 import dispatch as D
    n = B * S
    x = orc.rand_buf(n * d, 741, 2.0).reshape(n, d)
    res = orc.bf16_round(orc.rand_buf(n * d, 742, 1.0).reshape(n, d))
    gamma = 1.0 + orc.rand_buf(d, 743, 0.3)
    beta = orc.rand_buf(d, 744, 0.2)
    g16 = orc.bf16_round(orc.rand_buf(n * d, 745, 1.0).reshape(n, d))
    add_in = orc.rand_buf(n * d, 746, 1.0).reshape(n, d)
    add_bf = orc.bf16_round(orc.rand_buf(n * d, 747, 1.0).reshape(n, d))
    gp = [orc.bf16_round(orc.rand_buf(B * (S // c) * d, 750 + i, 1.0).reshape(B, S // c, d)) for i, c in enumerate(pools)]
    total = g16.reshape(B, S, d).copy()
    for g, c in zip(gp, pools):
        total += np.repeat(g, c, axis=1) / np.float32(c)
    xs = (x + res).astype(np.float32)
    out_r, mean_r, rstd_r = orc.layer_norm_forward(xs, gamma, beta, 1e-5)
    dx_r, dg_r, db_r = orc.layer_norm_backward(total.reshape(n, d), xs, gamma, mean_r, rstd_r)
    bf = torch.bfloat16
    xd, rd, gd, bd = _dev(x), _dev(res, bf), _dev(gamma), _dev(beta)
    o32 = torch.empty_like(xd); o16 = torch.empty(n, d, dtype=bf, device="cuda")
    mean = torch.empty(n, device="cuda"); rstd = torch.empty(n, device="cuda")
    D.call("nlh_layer_norm_residual_forward", x=xd, res=rd, res_is_bf16=1, gamma=gd, beta=bd, out_f32=o32,
           out_bf16=o16, mean_cache=mean, rstd_cache=rstd, n=n, d=d, eps=1e-5)
    assert max_abs(_np(o32), out_r) <= 2e-5
    assert rel_err(_np(o16), out_r) <= 1e-2
    gpd = [_dev(g, bf) for g in gp] + [None] * (3 - len(gp))
    cs = list(pools) + [1] * (3 - len(pools))
    dx = torch.empty_like(xd); dxb = torch.empty(n, d, dtype=bf, device="cuda")
    dgb = torch.zeros(2, d, device="cuda")
    D.call("nlh_layer_norm_backward_fused", d_out_f32=None, d_out_bf16=_dev(g16, bf),
           g0=gpd[0], c0=cs[0], g0_is_bf16=1, g1=gpd[1], c1=cs[1], g1_is_bf16=1, g2=gpd[2], c2=cs[2],
           g2_is_bf16=1, n_src=len(pools), seq=S, x=xd, res=rd, res_is_bf16=1, add_in=_dev(add_in), gamma=gd,
           mean_cache=mean, rstd_cache=rstd, d_x=dx, d_x_bf16=dxb, add_in_bf16=_dev(add_bf, bf),
           d_gamma=dgb[0], d_beta=dgb[1], n=n, d=d)
    assert rel_err(_np(dx), dx_r + add_in) <= 1e-4
    assert rel_err(_np(dxb), dx_r + add_bf) <= 1e-2
    assert rel_err(_np(dgb[0]), dg_r) <= 1e-4 and rel_err(_np(dgb[1]), db_r) <= 1e-4


@pytest.mark.parametrize("n,v", [(5, 37), (64, 8192), (3, 1000), (1, 1)])
def test_cross_entropy_drop_in_matches_oracle(orc, n, v):
    import torch
    from nl_hecate_b200 import dispatch as D
    logits = orc.rand_buf(n * v, 720 + n, 4.0).reshape(n, v)
    targets = (np.arange(n) * 7919 % v).astype(np.int32)
    if n >= 5:
        targets[1] = -1
        targets[3] = v            # invalid targets are skipped / their gradient rows zeroed
    s_r, cnt = orc.cross_entropy_sum(logits, targets)
    g_r = orc.cross_entropy_backward(logits, targets, 1.0 / max(cnt, 1))
    ld, td = _dev(logits), _dev(targets)
    loss = torch.full((1,), 123.0, device="cuda")     # the entry zeroes it
    D.call("cross_entropy_forward_cuda", logits=ld, target_ids=td, loss_out=loss, seq_len=n, vocab=v)
    assert abs(float(loss) - s_r) <= 1e-4 * max(1.0, abs(s_r))
    dl = torch.empty_like(ld)
    D.call("cross_entropy_backward_cuda", logits=ld, target_ids=td, d_logits=dl, seq_len=n, vocab=v,
           inv_count=1.0 / max(cnt, 1))
    assert max_abs(_np(dl), g_r) <= 2e-6


def test_cross_entropy_bf16_in_place(orc):
    import torch
    from nl_hecate_b200 import dispatch as D
    n, v = 96, 8192
    logits = orc.bf16_round(orc.rand_buf(n * v, 731, 6.0).reshape(n, v))
    targets = (np.arange(n) * 131 % v).astype(np.int32)
    targets[7] = -5
    s_r, cnt = orc.cross_entropy_sum(logits, targets)
    g_r = orc.cross_entropy_backward(logits, targets, 0.5 / cnt)
    ld, td = _dev(logits, torch.bfloat16), _dev(targets)
    acc = torch.zeros(1, device="cuda")
    cntd = torch.zeros(1, dtype=torch.int32, device="cuda")
    lse = torch.empty(n, device="cuda")
    D.call("nlh_cross_entropy_forward", logits=ld, logits_is_bf16=1, target_ids=td, loss_sum=acc,
           lse=lse, valid_count=cntd, n=n, vocab=v)
    assert int(cntd) == cnt
    assert abs(float(acc) - s_r) <= 2e-4 * abs(s_r)
    scale = torch.full((1,), 0.5, device="cuda")
    D.call("nlh_cross_entropy_backward", logits=ld, logits_is_bf16=1, target_ids=td, lse=lse,
           grad_scale=scale, d_logits=ld, n=n, vocab=v, inv_count=1.0 / cnt)
    got = _np(ld)
    assert np.all(got[7] == 0.0)
    assert max_abs(got, g_r) <= 1e-2 * np.abs(g_r).max()
    assert rel_err(got, g_r) <= 1e-2


def test_embedding_gather_and_scatter_add(orc):
    import torch
    from nl_hecate_b200 import dispatch as D
    vocab, d, n = 97, 512, 300
    w = orc.rand_buf(vocab * d, 741, 1.0).reshape(vocab, d)
    ids = (np.arange(n) ** 2 % 13).astype(np.int32)            # heavy repetition of a few rows
    g = orc.rand_buf(n * d, 742, 1.0).reshape(n, d)
    out = torch.empty(n, d, device="cuda")
    D.call("embedding_gather_cuda", w_embed=_dev(w), input_ids=_dev(ids), output=out, seq_len=n, d=d)
    assert np.array_equal(_np(out), orc.embedding_gather(w, ids))
    dw = torch.zeros(vocab, d, device="cuda")
    D.call("embedding_scatter_add_cuda", d_embedded=_dev(g), input_ids=_dev(ids), d_embed=dw, seq_len=n, d=d)
    assert rel_err(_np(dw), orc.embedding_scatter_add(g, ids, vocab)) <= 1e-5


def test_model_loss_with_fused_glue_matches_torch_glue():
    """Same parameters and batch: LayerNorm / cross-entropy kernels vs torch's, fp32 path."""
    import torch
    from nl_hecate_b200.stacked_mag import StackedMAG, StackedMAGConfig
    kw = dict(d_model=128, num_heads=2, n_blocks=2, k=2, chunk_sizes=(1, 8), seq_len=64, window=64,
              vocab=512, bf16=False)
    torch.manual_seed(0)
    tok = torch.randint(0, 512, (2, 64), device="cuda")
    tgt = torch.randint(0, 512, (2, 64), device="cuda")
    res = []
    for fused in (True, False):
        m = StackedMAG(StackedMAGConfig(fused_glue=fused, **kw), batch_per_rank=2)
        m.opt.g.zero_()
        loss = m.forward_backward(tok, tgt)
        res.append((float(loss), m.opt.g.clone()))
    assert abs(res[0][0] - res[1][0]) <= 1e-4 * abs(res[1][0])
    assert rel_err(_np(res[0][1]), _np(res[1][1])) <= 2e-3
