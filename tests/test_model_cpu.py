"""CPU tests of the host-side harness around the hot path: the stacked MAG model with the
hot-path operators replaced by plain-PyTorch statements, and its data-parallel gradient
exchange over gloo (world size 2)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from torch_ref import swa_ref, titans_memory_ref  # noqa: E402


def _tiny_cfg():
    from nl_hecate_b200.stacked_mag import StackedMAGConfig
    return StackedMAGConfig(d_model=32, num_heads=2, n_blocks=2, k=3, chunk_sizes=(1, 4, 16),
                            seq_len=16, window=8, vocab=64, bf16=False)


def _model(batch, seed=42):
    from nl_hecate_b200.stacked_mag import StackedMAG
    return StackedMAG(_tiny_cfg(), batch, device="cpu", seed=seed, memory_fn=titans_memory_ref,
                      swa_fn=swa_ref)


def _data(batch, seed=0):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, 64, (batch, 17), generator=g)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def test_forward_backward_fills_the_gradient_arena():
    m = _model(2)
    tok, tgt = _data(2)
    m.forward_backward(tok, tgt)      # first call: carried memories become non-zero
    m.opt.g.zero_()
    loss = m.forward_backward(tok, tgt)
    assert torch.isfinite(loss) and abs(float(loss) - torch.log(torch.tensor(64.0))) < 1.0
    # every parameter tensor received a gradient, written in place into the flat arena
    for i, n in enumerate(m.names):
        gv = m.opt.view(m.opt.g, i)
        assert gv.data_ptr() == m.g[n].data_ptr()
        assert torch.isfinite(gv).all(), n
        if n.endswith("l2.b_eta"):
            continue   # level 2 sees one pooled token per call and S0 = 0, so d_eta is exactly 0
        assert float(gv.abs().max()) > 0, n
    # carried memory was updated and is detached
    assert float(m.context[0][0].abs().max()) > 0 and not m.context[0][0].requires_grad


def test_pulse_and_level_activity():
    m = _model(1)
    assert m.pulse() == [True, True, True]          # seq_len 16 >= every chunk size
    m.cfg.seq_len = 2
    m.global_step = 3
    assert m.pulse() == [True, False, False]        # step % cs != 0 and seq_len < cs
    m.global_step = 4
    assert m.pulse() == [True, True, False]


def test_param_count_formula():
    m = _model(1)
    d, v, k, nb = 32, 64, 3, 2
    per_level = 3 * d * d + 3 * 2 * d + 3
    want = 2 * v * d + 2 * d + nb * (4 * d * d + 4 * d + k + k * per_level)
    assert m.n_params() == want


def _dp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    tok, tgt = _data(4)
    m = _model(2)
    lo = rank * 2
    m.forward_backward(tok[lo:lo + 2], tgt[lo:lo + 2])
    m.sync_gradients(None, world)
    one = m.opt.g.clone()
    # the same exchange in per-block buckets issued from autograd hooks during the backward
    m2 = _model(2)
    m2.forward_backward(tok[lo:lo + 2], tgt[lo:lo + 2], None, world)
    assert m2._grads_synced
    m2.sync_gradients(None, world)          # no second exchange
    assert torch.allclose(m2.opt.g, one, atol=1e-9, rtol=1e-6)
    assert sorted(m2._last_buckets) == sorted(m2._bucket_order())
    q.put((rank, one))
    dist.barrier()
    dist.destroy_process_group()


def test_data_parallel_gradients_match_global_batch():
    """Batch shard + one all-reduce(SUM)/world over the arena == gradients of the global batch
    (core/src/distributed.rs:121-150 semantics; inner-loop state stays rank-local)."""
    world, port = 2, 29731
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_dp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    tok, tgt = _data(4)
    ref = _model(4)
    ref.forward_backward(tok, tgt)
    assert torch.allclose(got[0], got[1], atol=0, rtol=0)          # ranks agree bit for bit
    assert torch.allclose(got[0], ref.opt.g, atol=2e-6, rtol=1e-4)  # and match the global batch


def test_sync_gradients_world1_is_a_no_op():
    m = _model(1)
    tok, tgt = _data(1)
    m.forward_backward(tok, tgt)
    before = m.opt.g.clone()
    m.sync_gradients(None, 1)
    assert torch.equal(before, m.opt.g)


def test_harness_forward_matches_an_independent_float64_statement():
    """The stacked harness (plain-PyTorch operators, fp32) against tests/refmath.py's float64
    numpy statement of the same block composition, over two consecutive calls so that the
    carried memories are non-zero in the second one."""
    import numpy as np
    from refmath import stacked_mag_loss64
    m = _model(2, seed=11)
    cfg = m.cfg
    # make every branch matter: random LayerNorm affine terms, level weights and gate biases
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for n, w in m.p.items():
            base = n.split(".")[-1]
            if base.endswith("gamma"):
                w.add_(0.2 * torch.randn(w.shape, generator=g))
            elif base.endswith("beta") or base == "alpha_mem":
                w.add_(0.3 * torch.randn(w.shape, generator=g))
            elif base == "b_theta":
                w.fill_(-1.0)
            elif base == "b_alpha":
                w.fill_(-2.0)
    params = {n: w.detach().numpy().astype(np.float64) for n, w in m.p.items()}
    cfgd = dict(d_model=cfg.d_model, num_heads=cfg.num_heads, n_blocks=cfg.n_blocks, k=cfg.k,
                chunk_sizes=cfg.chunk_sizes, window=cfg.window, exact_levels=cfg.exact_levels)
    ctx = [[np.zeros((2 * cfg.num_heads, cfg.head_dim ** 2)) for _ in range(cfg.k)] for _ in range(cfg.n_blocks)]
    for call in range(2):
        tok, tgt = _data(2, seed=call)
        with torch.no_grad():
            got = float(m.forward(tok, tgt))
        want = stacked_mag_loss64(params, cfgd, tok.numpy(), tgt.numpy(), ctx)
        assert abs(got - want) <= 2e-4 * abs(want), (call, got, want)
    for b in range(cfg.n_blocks):
        for l in range(cfg.k):
            a, r = m.context[b][l].numpy(), ctx[b][l]
            assert np.abs(a - r).max() <= 1e-4 * max(np.abs(r).max(), 1e-9), (b, l)
