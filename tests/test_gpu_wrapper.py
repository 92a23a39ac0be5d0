"""GPU: fused rule-wrapper kernels (level prep, MAG combine, pool-to-heads) through the C ABI
vs the same math written with PyTorch ops and autograd (fp32, relative error <= 1e-4)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-12))


def _torch_level_prep(kvq, w_gates, b_a, b_t, b_e, H):
    B, sf, d3 = kvq.shape
    d = d3 // 3
    hd = d // H
    k, v, q = kvq.float().split(d, dim=-1)
    k = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-8)
    q = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-8)
    pre = torch.cat([k, v], -1) @ w_gates.t()
    al = torch.sigmoid(pre[..., 0] + b_a)
    th = F.softplus(pre[..., 1] + b_t)
    et = torch.sigmoid(pre[..., 2] + b_e)
    heads = lambda t: t.reshape(B, sf, H, hd).permute(0, 2, 1, 3).reshape(B * H, sf, hd)
    bro = lambda t: t.unsqueeze(1).expand(B, H, sf).reshape(B * H, sf)
    return heads(k), heads(v), heads(q), bro(al), bro(th), bro(et)


@pytest.mark.parametrize("B,sf,d,H", [(2, 5, 128, 2), (3, 33, 512, 8), (1, 1, 64, 1), (2, 40, 192, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_level_prep_forward_backward(B, sf, d, H, dtype):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import _LevelPrep
    g = torch.Generator(device="cuda").manual_seed(B * 100 + sf)
    r = lambda *sh: torch.randn(*sh, generator=g, device="cuda")
    kvq = r(B, sf, 3 * d).to(dtype)
    w = 0.05 * r(3, 2 * d)
    ba, bt, be = r(1), r(1) - 2.0, r(1)
    ups = [r(B * H, sf, d // H) for _ in range(3)] + [r(B * H, sf) for _ in range(3)]

    def run(fn):
        leaves = [t.clone().requires_grad_(True) for t in (kvq, w, ba, bt, be)]
        outs = fn(*leaves)
        loss = sum((o * u).sum() for o, u in zip(outs, ups))
        loss.backward()
        return [o.detach() for o in outs], [t.grad for t in leaves]

    o1, g1 = run(lambda kvq_, w_, a_, t_, e_: _LevelPrep.apply(kvq_, w_, a_, t_, e_, H))
    o2, g2 = run(lambda kvq_, w_, a_, t_, e_: _torch_level_prep(kvq_, w_, a_, t_, e_, H))
    for a, b in zip(o1, o2):
        assert _rel(a, b) <= 1e-5
    tol = 1e-4 if dtype == torch.float32 else 1e-2   # d_kvq is rounded to bf16 in that mode
    for name, a, b in zip(("d_kvq", "d_w_gates", "d_b_alpha", "d_b_theta", "d_b_eta"), g1, g2):
        assert a.dtype == b.dtype
        assert _rel(a, b) <= (tol if name == "d_kvq" else 1e-4), (name, _rel(a, b))


def _torch_combine(x, ap, wts, pools, H, ys):
    B, S, d = x.shape
    hd = d // H
    y = 0
    for l, (yl, c) in enumerate(zip(ys, pools)):
        sf = S // c
        full = yl.view(B, H, sf, hd).permute(0, 2, 1, 3).reshape(B, sf, d).repeat_interleave(c, dim=1)
        y = y + wts[l] * full
    return x + ap.float() * torch.sigmoid(y)


@pytest.mark.parametrize("B,S,d,H,pools", [(2, 16, 128, 2, (1, 4, 16)), (2, 64, 512, 8, (1, 8, 64, 64)),
                                           (1, 8, 64, 1, (1,)), (3, 24, 192, 3, (1, 2, 8, 24))])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mag_combine_forward_backward(B, S, d, H, pools, dtype):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import _MagCombine
    g = torch.Generator(device="cuda").manual_seed(S + d)
    r = lambda *sh: torch.randn(*sh, generator=g, device="cuda")
    x, ap = r(B, S, d), r(B, S, d).to(dtype)
    alpha_mem = r(len(pools))
    ys = [r(B * H, S // c, d // H) for c in pools]
    up = r(B, S, d)

    def run(fn):
        leaves = [t.clone().requires_grad_(True) for t in [x, ap, alpha_mem] + ys]
        wts = torch.softmax(leaves[2], 0)
        out = fn(leaves[0], leaves[1], wts, leaves[3:])
        (out * up).sum().backward()
        return out.detach(), [t.grad for t in leaves]

    o1, g1 = run(lambda x_, ap_, w_, ys_: _MagCombine.apply(x_, ap_, w_, pools, H, None, None, *ys_))
    o2, g2 = run(lambda x_, ap_, w_, ys_: _torch_combine(x_, ap_, w_, pools, H, ys_))
    assert _rel(o1, o2) <= 1e-5
    names = ["d_x", "d_attn_proj", "d_alpha_mem"] + [f"d_y{l}" for l in range(len(pools))]
    for name, a, b in zip(names, g1, g2):
        tol = 1e-2 if (name == "d_attn_proj" and dtype == torch.bfloat16) else 1e-4
        assert _rel(a, b) <= tol, (name, _rel(a, b))


def test_partial_row_finishers_accumulate_into_gradient_buffers():
    """nlh_gate_grad_finish and nlh_level_weight_grad_finish: column sums of the partial rows,
    added to what the gradient buffers already hold; the level weights go through the softmax
    adjoint."""
    from nl_hecate_b200 import dispatch as D
    g = torch.Generator().manual_seed(3)
    for rows, d in [(1, 64), (37, 512), (300, 128)]:
        dwp = torch.randn(rows, 3, 2 * d, generator=g).cuda()
        dbp = torch.randn(rows, 3, generator=g).cuda()
        gw = torch.randn(3, 2 * d, generator=g).cuda()
        gb = [torch.randn(1, generator=g).cuda() for _ in range(3)]
        want_w = gw.double() + dwp.double().sum(0)
        want_b = [gb[i].double() + dbp.double().sum(0)[i] for i in range(3)]
        D.call("nlh_gate_grad_finish", dw_partial=dwp, db_partial=dbp, rows=rows, d_model=d,
               g_w_gates=gw, g_b_alpha=gb[0], g_b_theta=gb[1], g_b_eta=gb[2])
        assert float((gw.double() - want_w).abs().max()) <= 1e-4 * float(want_w.abs().max())
        for i in range(3):
            assert abs(float(gb[i]) - float(want_b[i])) <= 1e-4 * max(1.0, abs(float(want_b[i])))
    for rows, k in [(1, 1), (1184, 4), (50, 3)]:
        dwp = torch.randn(rows, 4, generator=g).cuda()
        logits = torch.randn(k, generator=g).cuda().requires_grad_(True)
        w = torch.softmax(logits, 0)
        (w * dwp[:, :k].sum(0)).sum().backward()
        gl = torch.full((k,), 0.25, device="cuda")
        D.call("nlh_level_weight_grad_finish", dw_partial=dwp, rows=rows, k=k, level_weights=w.detach().contiguous(),
               g_logits=gl)
        assert float((gl - 0.25 - logits.grad).abs().max()) <= 1e-4 * max(1.0, float(logits.grad.abs().max()))


def test_wrapper_rejects_unsupported_shapes():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch as D
    z = torch.zeros(16, device="cuda")
    with pytest.raises(RuntimeError):   # head_dim 6 is not a multiple of 4
        D.call("nlh_pool_to_heads", d_ycomb=z, level_weights=z, level=0, pool=1, dy_ph=z, sum_out=None,
               batch=1, seq=1, d_model=12, num_heads=2)
    with pytest.raises(RuntimeError):   # 6 source rows cannot be pooled by 4
        D.call("nlh_pool_heads", src_sums=z, level_weights=z, level=1, factor=4, dy_ph=z, sum_out=None,
               rows=1, src_seq=6, head_dim=4)


def test_hierarchical_pooling_equals_direct_pooling():
    """Pooling by 64 from the by-8 sums gives what a direct pass over d_ycomb gives."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200 import dispatch as D
    B, S, d, H = 3, 128, 64, 4
    g = torch.Generator(device="cuda").manual_seed(5)
    dyc = torch.randn(B, S, d, device="cuda", generator=g)
    wts = torch.tensor([0.1, 0.2, 0.3, 0.4], device="cuda")
    hd = d // H
    fine = torch.empty(B * H, S // 8, hd, device="cuda")
    sums = torch.empty_like(fine)
    D.call("nlh_pool_to_heads", d_ycomb=dyc, level_weights=wts, level=1, pool=8, dy_ph=fine, sum_out=sums,
           batch=B, seq=S, d_model=d, num_heads=H)
    ref8 = dyc.view(B, S // 8, 8, H, hd).sum(2).permute(0, 2, 1, 3).reshape(B * H, S // 8, hd)
    assert _rel(sums, ref8) <= 1e-6 and _rel(fine, 0.2 * ref8) <= 1e-6
    direct = torch.empty(B * H, S // 64, hd, device="cuda")
    D.call("nlh_pool_to_heads", d_ycomb=dyc, level_weights=wts, level=2, pool=64, dy_ph=direct, sum_out=None,
           batch=B, seq=S, d_model=d, num_heads=H)
    chained = torch.empty_like(direct)
    D.call("nlh_pool_heads", src_sums=sums, level_weights=wts, level=2, factor=8, dy_ph=chained, sum_out=None,
           rows=B * H, src_seq=S // 8, head_dim=hd)
    assert _rel(chained, direct) <= 1e-5


@pytest.mark.parametrize("pools,dtype", [((8, 64, 512), torch.bfloat16), ((2, 8, 24), torch.float32),
                                         ((4,), torch.float32), ((2, 3, 4, 12), torch.bfloat16)])
def test_pool_levels_forward_backward(pools, dtype):
    """Mean pooling of the level inputs and its fused adjoint vs torch."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from nl_hecate_b200.stacked_mag import _PoolLevels
    B, d = 2, 64
    S = 512 if 512 in pools else 48
    g = torch.Generator(device="cuda").manual_seed(S)
    x1 = torch.randn(B, S, d, device="cuda", generator=g, requires_grad=True)
    x2 = x1.detach().clone().requires_grad_(True)
    outs = _PoolLevels.apply(x1, pools, dtype == torch.bfloat16)
    refs = [x2.view(B, S // c, c, d).mean(2).to(dtype) for c in pools]
    ws = [torch.randn(o.shape, device="cuda", generator=g) for o in refs]
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    for o, r in zip(outs, refs):
        assert o.dtype == dtype and _rel(o, r) <= tol
    sum((o.float() * w).sum() for o, w in zip(outs, ws)).backward()
    sum((r.float() * w).sum() for r, w in zip(refs, ws)).backward()
    assert _rel(x1.grad, x2.grad) <= tol
