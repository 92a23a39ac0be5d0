"""Stacked Titans-LMM + MAG + SWA model with CMS levels: the caller of the hot path.

Host-side harness standing in for the reference's GPU-resident driver
(core/src/gpu_stacked_forward.rs:1263-2038 forward_sequence, gpu_forward.rs:1197-1540
gpu_memory_forward, gpu_stacked_backward.rs, gpu_stacked_optimizer.rs:522-700). The hot-path
operators — memory-rule kernel pairs, SWA forward/backward, the AdamW step — and the glue
around them (rule wrapper, level pooling, MAG gating, LayerNorm, cross-entropy) are this
library's CUDA kernels behind the C ABI, registered as opaque blocks of PyTorch's tape; the
dense projections and the embedding stay cuBLAS / PyTorch. With fused_glue = False (and on
CPU) the glue runs as plain PyTorch operators, which the tests use as the second statement.

Block (MAG composition), per core/src/gpu_stacked_forward.rs:1656-1960:
    h        = LN_attn(x)
    q,k,v    = h W_q^T, h W_k^T, h W_v^T           (bf16)
    attn     = SWA(q,k,v)  ;  attn_proj = attn W_o^T ; res1 = x + attn_proj
    m_in     = LN_mem(res1)
    level l  : x_l = mean_pool(m_in, c_l)            (c_l = chunk size of the level)
               k,v,q = x_l W_{k,v,q}^T ; k,q L2-normalised over d_model
               alpha = sigmoid([k;v].w_a + b_a), theta = softplus([k;v].w_t + b_t),
               eta = sigmoid([k;v].w_e + b_e)        (one gate per token, shared by heads)
               y_l  = TitansLMM per head on [B*H, s/c_l, hd]: level 0 exact per-token rule,
                      levels >= 1 frozen-M0 chunkwise rule; M carried across steps, S0 = 0
               y_l upsampled by repetition to full resolution
    y        = sum_l softmax(alpha_mem)_l y_l
    out      = x + attn_proj * sigmoid(y)            (second residual adds to the block INPUT)
Final LayerNorm, unembedding (logits = x W_unembed, W_unembed [d, vocab]), cross-entropy.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from . import dispatch as D
from .optimizer import FlatAdamW

B_ALPHA = (3.0, 4.0, 4.5, 5.0, 5.5, 6.0)      # core/src/model.rs:1081-1093
B_THETA = (-4.6, -5.6, -6.6, -7.6, -8.6, -9.6)  # core/src/model.rs:1095-1109
B_ETA = (1.5, 2.0, 2.5, 3.0, 3.5, 4.0)        # core/src/model.rs:1111-1122


@dataclass
class StackedMAGConfig:
    d_model: int = 512
    num_heads: int = 8
    n_blocks: int = 4
    k: int = 4
    chunk_sizes: tuple = (1, 8, 64, 512)
    seq_len: int = 512
    window: int = 512
    vocab: int = 8192
    bf16: bool = True                 # bf16 activations for SWA and the dense projections
    exact_levels: tuple = (0,)        # tape strategy: level 0 exact, others frozen-M0 (proxy)
    exact_checkpoint: int = 0         # > 0: exact levels keep a checkpoint every this many tokens and
                                      # recompute the windows in the backward (less memory, more time)
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    tie_embeddings: bool = True
    fused_glue: bool = True           # fused CUDA rule wrapper / MAG combine (CUDA only)
    level_streams: bool = True        # run CMS levels >= 1 on side streams next to level 0
    overlap_grad_sync: bool = True    # data-parallel: all-reduce each block's gradients under the rest of the backward

    @property
    def head_dim(self):
        return self.d_model // self.num_heads


class _TitansMemory(torch.autograd.Function):
    """Per-head Titans LMM over [N, S, hd] (N = batch*heads) through the C ABI.
    chunk == 0: exact rule (titans_forward/backward_f32_cuda, M trajectory only);
    chunk > 0 : frozen-M0 chunkwise rule — chunk-boundary states and the chunk-parallel kernels
    (titans_chunkwise_*_f32_cuda) for chunks of 16 tokens and more; for shorter chunks (the pooled
    CMS levels see 64, 8 and 1 tokens) every state is stored and the backward streams them
    (nlh_rule_forward / nlh_rule_backward with interval = 1). One-token chunks stay on the
    chunk-boundary entries: their stored S_0 = 0 gives the exactly-zero d_eta of a level that sees
    a single token per call, which the M-difference form only reaches to rounding."""

    STREAM_BELOW = 16        # chunks shorter than this take the full-trajectory frozen pair ...
    # ... unless the problems (batch x heads) number at most half the SMs: level 0 is then split over
    # two CTAs per problem and fills the GPU, and the lighter chunk-boundary kernels disturb it less
    # next to it (measured at 64 problems: 4.89 ms per step against 5.26 ms)
    STREAM_MIN_PROBLEMS = None

    @staticmethod
    def _stream_ok(k, chunk):
        if not (1 < chunk < _TitansMemory.STREAM_BELOW and k.shape[-1] in (32, 64)):
            return False
        lo = _TitansMemory.STREAM_MIN_PROBLEMS
        if lo is None:
            lo = torch.cuda.get_device_properties(k.device).multi_processor_count // 2 + 1
        return k.shape[0] >= lo

    _ZEROS = {}

    @staticmethod
    def forward(ctx, k, v, q, alpha, theta, eta, m0, chunk, slot=0, carry=None, ckpt=0):
        # momentum restarts every call (gpu_forward.rs:1516-1517): S_0 = 0, a read-only buffer that
        # is created once per shape instead of being filled every call
        key = (tuple(m0.shape), m0.device)
        s0 = _TitansMemory._ZEROS.get(key)
        if s0 is None:
            s0 = _TitansMemory._ZEROS[key] = torch.zeros_like(m0)
        ctx.slot = slot
        with D.workspace_slot(slot):
            return _TitansMemory._forward(ctx, k, v, q, alpha, theta, eta, m0, s0, chunk, carry, ckpt)

    @staticmethod
    def _forward(ctx, k, v, q, alpha, theta, eta, m0, s0, chunk, carry=None, ckpt=0):
        ctx.stream = _TitansMemory._stream_ok(k, chunk)
        ctx.ckpt = ckpt if chunk == 0 else 0
        if chunk == 0 and ckpt > 0:
            # exact rule, checkpoints only (reference semantics core/src/cuda_ffi.rs:230,262): the
            # trajectory shrinks by the interval, the backward recomputes each window
            ms, ss, y = D.rule_forward(1, k, v, q, alpha, theta, eta, m0, s0, ckpt, 0)
            ctx.save_for_backward(k, v, q, alpha, theta, eta, ms, ss)
        elif chunk == 0:
            # M trajectory only: the backward derives S_t = M_t - (1-alpha_{t-1}) M_{t-1}
            ms, ss, y = D.titans_forward_dd(k, v, q, alpha, theta, eta, m0, s0, store_s=False)
            ctx.save_for_backward(k, v, q, alpha, theta, eta, ms)
        elif ctx.stream:
            ms, y = D.titans_frozen_stream_forward(k, v, q, alpha, theta, eta, m0, s0, chunk)
            ctx.save_for_backward(k, v, q, alpha, theta, eta, ms)
        else:
            ms, ss, y = D.titans_chunkwise_forward_dd(k, v, q, alpha, theta, eta, m0, s0, chunk)
            ctx.save_for_backward(k, v, q, alpha, theta, eta, ms, ss)
        ctx.chunk = chunk
        if carry is not None:
            # the carried memory is updated in place from the last stored state (one strided copy;
            # the kernels have read m0 by then, stream order), no separate m_final tensor
            carry.copy_(ms[:, -1])
            return y, None
        m_final = ms[:, -1].clone()
        ctx.mark_non_differentiable(m_final)
        return y, m_final

    @staticmethod
    def backward(ctx, dy, _dm):
        dy = dy.contiguous()
        with D.workspace_slot(ctx.slot):
            if ctx.ckpt > 0:
                k, v, q, alpha, theta, eta, ms, ss = ctx.saved_tensors
                g = D.rule_backward(1, k, v, q, alpha, theta, eta, ms, ss, dy, ctx.ckpt, 0)
            elif ctx.chunk == 0:
                k, v, q, alpha, theta, eta, ms = ctx.saved_tensors
                g = D.titans_backward_dd(k, v, q, alpha, theta, eta, ms, None, dy, want_initial=False)
            elif ctx.stream:
                k, v, q, alpha, theta, eta, ms = ctx.saved_tensors
                g = D.titans_frozen_stream_backward(k, v, q, alpha, theta, eta, ms, dy, ctx.chunk,
                                                    want_initial=False)
            else:
                k, v, q, alpha, theta, eta, ms, ss = ctx.saved_tensors
                g = D.titans_chunkwise_backward_dd(k, v, q, alpha, theta, eta, ms, ss, dy, ctx.chunk,
                                                   want_initial=False)
        return (g["d_k"], g["d_v"], g["d_q"], g["d_alpha"], g["d_theta"], g["d_eta"], None, None, None,
                None, None)


class _SWA(torch.autograd.Function):
    """Sliding-window attention over [B, S, H*hd]: bf16 inputs run the tensor-core pair
    (nlh_swa_forward / nlh_swa_backward), fp32 inputs the fp32 pair (nlh_swa_forward_f32 /
    nlh_swa_backward_f32)."""

    @staticmethod
    def forward(ctx, q, k, v, num_heads, head_dim, window):
        f32 = q.dtype == torch.float32
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse = (D.swa_forward_f32 if f32 else D.swa_forward_lse)(q, k, v, num_heads, head_dim, window)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (num_heads, head_dim, window, f32)
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse = ctx.saved_tensors
        nh, hd, w, f32 = ctx.cfg
        bwd = D.swa_backward_f32 if f32 else D.swa_backward_lse
        dq, dk, dv = bwd(q, k, v, out, lse, d_out.float().contiguous(), nh, hd, w)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None


class _SWAPacked(torch.autograd.Function):
    """Sliding-window attention straight on the projection output qkv [B, S, 3*H*hd] bf16
    (nlh_swa_forward_packed / nlh_swa_backward_packed): no q/k/v split copies, bf16 gradient in,
    packed bf16 gradient out."""

    @staticmethod
    def forward(ctx, qkv, num_heads, head_dim, window):
        qkv = qkv.contiguous()
        B, S, _ = qkv.shape
        out = torch.empty(B, S, num_heads * head_dim, dtype=torch.bfloat16, device=qkv.device)
        lse = torch.empty(B, num_heads, S, dtype=torch.float32, device=qkv.device)
        D.call("nlh_swa_forward_packed", qkv=qkv, out=out, lse=lse, seq_len=S, num_heads=num_heads,
               head_dim=head_dim, window_size=window, batch_size=B, n_persistent=0)
        ctx.save_for_backward(qkv, out, lse)
        ctx.cfg = (num_heads, head_dim, window)
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, out, lse = ctx.saved_tensors
        nh, hd, w = ctx.cfg
        B, S, _ = qkv.shape
        d_qkv = torch.empty_like(qkv)
        D.call("nlh_swa_backward_packed", qkv=qkv, out=out, lse=lse,
               d_attn_out=d_out.to(torch.bfloat16).contiguous(), d_qkv=d_qkv, seq_len=S, num_heads=nh,
               head_dim=hd, window_size=w, batch_size=B, n_persistent=0)
        return d_qkv, None, None, None


class _LevelPrep(torch.autograd.Function):
    """kvq [B, s, 3d] (k|v|q rows from the projection GEMM) -> per-head k,v,q and gates
    (nlh_level_prep_forward / _backward): L2 norm of k,q over d_model, the three gates, head
    split, and in backward the gate/L2-norm/transposes adjoints plus gate weight gradients."""

    @staticmethod
    def forward(ctx, kvq, w_gates, b_alpha, b_theta, b_eta, num_heads, slot=0, grads=None):
        """grads = (g_w_gates, g_b_alpha, g_b_theta, g_b_eta): gradient buffers the backward adds
        the four parameter gradients into (nlh_gate_grad_finish); it then returns none for them."""
        kvq = kvq.contiguous()
        ctx.slot = slot
        ctx.grads = grads
        B, sf, d3 = kvq.shape
        d, H = d3 // 3, num_heads
        hd, dev = d // H, kvq.device
        f32 = lambda *sh: torch.empty(*sh, dtype=torch.float32, device=dev)
        k_ph, v_ph, q_ph = f32(B * H, sf, hd), f32(B * H, sf, hd), f32(B * H, sf, hd)
        al, th, et = f32(B * H, sf), f32(B * H, sf), f32(B * H, sf)
        kn, qn = f32(B * sf), f32(B * sf)
        is_bf16 = int(kvq.dtype == torch.bfloat16)
        D.call("nlh_level_prep_forward", kvq=kvq, kvq_is_bf16=is_bf16, w_gates=w_gates,
               b_alpha=b_alpha, b_theta=b_theta, b_eta=b_eta, k_ph=k_ph, v_ph=v_ph, q_ph=q_ph,
               alpha_ph=al, theta_ph=th, eta_ph=et, k_norm=kn, q_norm=qn, batch=B, seq=sf,
               d_model=d, num_heads=H)
        ctx.save_for_backward(k_ph, v_ph, q_ph, al, th, et, kn, qn, w_gates)
        ctx.meta = (B, sf, d, H, is_bf16, kvq.dtype)
        return k_ph, v_ph, q_ph, al, th, et

    @staticmethod
    def backward(ctx, dk, dv, dq, da, dt, de):
        k_ph, v_ph, q_ph, al, th, et, kn, qn, w_gates = ctx.saved_tensors
        B, sf, d, H, is_bf16, dtype = ctx.meta
        dev = k_ph.device
        z = lambda g, like: torch.zeros_like(like) if g is None else g.contiguous()
        dk, dv, dq = z(dk, k_ph), z(dv, v_ph), z(dq, q_ph)
        da, dt, de = z(da, al), z(dt, th), z(de, et)
        rows = int(D.ffi.lib().nlh_level_prep_partial_rows(B * sf))
        d_kvq = torch.empty(B, sf, 3 * d, dtype=dtype, device=dev)
        dwp = torch.empty(rows, 3, 2 * d, dtype=torch.float32, device=dev)
        dbp = torch.empty(rows, 3, dtype=torch.float32, device=dev)
        with D.workspace_slot(ctx.slot):
            D.call("nlh_level_prep_backward", k_ph=k_ph, v_ph=v_ph, q_ph=q_ph, alpha_ph=al, theta_ph=th,
                   eta_ph=et, k_norm=kn, q_norm=qn, dk_ph=dk, dv_ph=dv, dq_ph=dq, dalpha_ph=da,
                   dtheta_ph=dt, deta_ph=de, w_gates=w_gates, d_kvq=d_kvq, kvq_is_bf16=is_bf16,
                   dw_partial=dwp, db_partial=dbp, batch=B, seq=sf, d_model=d, num_heads=H)
            if ctx.grads is not None:
                gw, ga, gt, ge = ctx.grads
                D.call("nlh_gate_grad_finish", dw_partial=dwp, db_partial=dbp, rows=rows, d_model=d,
                       g_w_gates=gw, g_b_alpha=ga, g_b_theta=gt, g_b_eta=ge)
                return d_kvq, None, None, None, None, None, None, None
        dw = dwp.sum(0)
        db = dbp.sum(0)
        return d_kvq, dw, db[0:1], db[1:2], db[2:3], None, None, None


class _MagCombine(torch.autograd.Function):
    """out = x + attn_proj * sigmoid(sum_l w_l upsample(y_l)) on per-head level outputs
    (nlh_mag_combine_forward / _backward + nlh_pool_to_heads)."""
    ROWS = 148 * 8

    @staticmethod
    def forward(ctx, x, attn_proj, wts, pools, num_heads, g_logits, fan, *ys):
        """wts = softmax(alpha_mem). g_logits None: wts is a tensor of the graph and receives its
        gradient. g_logits = gradient buffer of alpha_mem: wts was computed outside the graph, the
        backward adds the softmax adjoint into g_logits (nlh_level_weight_grad_finish).
        fan (dict or None): the block's gradient fan-in. When given, the backward does NOT return
        the gradients of x and attn_proj; it leaves them in fan["c_dx"], fan["c_dap"] for the
        block's memory LayerNorm backward, whose kernel adds them to its own (those two tensors have
        other consumers in the block, and the sums would otherwise be separate passes)."""
        ctx.g_logits = g_logits
        ctx.fan = fan
        x, attn_proj, wts = x.contiguous(), attn_proj.contiguous(), wts.contiguous().float()
        B, S, d = x.shape
        k = len(ys)
        ys = [y.contiguous() for y in ys]
        yp = ys + [None] * (4 - k)
        cp = list(pools) + [1] * (4 - k)
        out = torch.empty_like(x)
        is_bf16 = int(attn_proj.dtype == torch.bfloat16)
        D.call("nlh_mag_combine_forward", x=x, attn_proj=attn_proj, attn_is_bf16=is_bf16,
               level_weights=wts, y0=yp[0], y1=yp[1], y2=yp[2], y3=yp[3], c0=cp[0], c1=cp[1],
               c2=cp[2], c3=cp[3], k=k, out=out, batch=B, seq=S, d_model=d, num_heads=num_heads)
        ctx.save_for_backward(attn_proj, wts, *ys)
        ctx.meta = (B, S, d, num_heads, k, cp, is_bf16)
        return out

    @staticmethod
    def backward(ctx, d_out):
        attn_proj, wts, *ys = ctx.saved_tensors
        B, S, d, H, k, cp, is_bf16 = ctx.meta
        d_out = d_out.contiguous()
        dev = d_out.device
        yp = list(ys) + [None] * (4 - k)
        d_ap = torch.empty_like(attn_proj)
        d_yc = torch.empty(B, S, d, dtype=torch.float32, device=dev)
        rows = _MagCombine.ROWS
        dwp = torch.empty(rows, 4, dtype=torch.float32, device=dev)
        dys = [torch.empty_like(ys[l]) for l in range(k)]
        direct = [dys[l] if cp[l] == 1 else None for l in range(k)] + [None] * (4 - k)
        D.call("nlh_mag_combine_backward", d_out=d_out, attn_proj=attn_proj, attn_is_bf16=is_bf16,
               level_weights=wts, y0=yp[0], y1=yp[1], y2=yp[2], y3=yp[3], c0=cp[0], c1=cp[1],
               c2=cp[2], c3=cp[3], k=k, d_attn_proj=d_ap, d_ycomb=d_yc, dw_partial=dwp,
               n_partial_rows=rows, dy0=direct[0], dy1=direct[1], dy2=direct[2], dy3=direct[3],
               batch=B, seq=S, d_model=d, num_heads=H)
        if ctx.g_logits is not None:
            D.call("nlh_level_weight_grad_finish", dw_partial=dwp, rows=rows, k=k, level_weights=wts,
                   g_logits=ctx.g_logits)
            d_wts = None
        else:
            d_wts = dwp.sum(0)[:k]
        # pooled levels, finest first; a level whose pool factor is a multiple of the previous
        # pooled level's is reduced from that level's unscaled sums instead of from d_ycomb
        order = sorted((l for l in range(k) if cp[l] != 1), key=lambda l: cp[l])
        prev = None                                        # (pool factor, unscaled sums)
        for i, l in enumerate(order):
            later = any(cp[m] % cp[l] == 0 for m in order[i + 1:])
            sums = torch.empty_like(dys[l]) if later else None
            if prev is not None and cp[l] % prev[0] == 0:
                D.call("nlh_pool_heads", src_sums=prev[1], level_weights=wts, level=l,
                       factor=cp[l] // prev[0], dy_ph=dys[l], sum_out=sums, rows=B * H,
                       src_seq=S // prev[0], head_dim=d // H)
            else:
                D.call("nlh_pool_to_heads", d_ycomb=d_yc, level_weights=wts, level=l, pool=cp[l],
                       dy_ph=dys[l], sum_out=sums, batch=B, seq=S, d_model=d, num_heads=H)
            if sums is not None:
                prev = (cp[l], sums)
        if ctx.fan is not None:
            ctx.fan["c_dx"], ctx.fan["c_dap"] = d_out, d_ap
            return (None, None, d_wts, None, None, None, None, *dys)
        return (d_out, d_ap, d_wts, None, None, None, None, *dys)


class _PoolLevels(torch.autograd.Function):
    """Inputs of the pooled CMS levels: mean over c_l consecutive tokens of m_in [B, S, d] for each
    pool factor (ascending), coarser levels reduced from the finer level's sums when divisible
    (nlh_mean_pool); the backward adds all levels' upsampled gradients in one pass
    (nlh_unpool_sum). Outputs are bf16 when out_bf16 (they feed the projection GEMM)."""

    @staticmethod
    def forward(ctx, m_in, pools, out_bf16):
        m_in = m_in.contiguous()
        B, S, d = m_in.shape
        dt = torch.bfloat16 if out_bf16 else torch.float32
        outs, prev = [], None                       # prev = (pool factor, unscaled sums)
        for i, c in enumerate(pools):
            later = any(c2 % c == 0 for c2 in pools[i + 1:])
            out = torch.empty(B, S // c, d, dtype=dt, device=m_in.device)
            sums = torch.empty(B, S // c, d, dtype=torch.float32, device=m_in.device) if later else None
            if prev is not None and c % prev[0] == 0:
                src, f = prev[1], c // prev[0]
            else:
                src, f = m_in, c
            D.call("nlh_mean_pool", src=src, factor=f, scale=1.0 / c, out=out, out_is_bf16=int(out_bf16),
                   sum_out=sums, rows_out=B * (S // c), d_model=d)
            if sums is not None:
                prev = (c, sums)
            outs.append(out)
        ctx.meta = (B, S, d, tuple(pools))
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        B, S, d, pools = ctx.meta
        dev = next(g for g in grads if g is not None).device
        out = torch.empty(B, S, d, dtype=torch.float32, device=dev)
        src = [(g.contiguous(), c) for g, c in zip(grads, pools) if g is not None]
        first = True
        for i in range(0, len(src), 3):              # three levels per pass
            part = src[i:i + 3] + [(None, 1)] * (3 - len(src[i:i + 3]))
            dst = out if first else torch.empty_like(out)
            D.call("nlh_unpool_sum", g0=part[0][0], c0=part[0][1], g0_is_bf16=int(part[0][0].dtype == torch.bfloat16),
                   g1=part[1][0], c1=part[1][1], g1_is_bf16=int(part[1][0] is not None and part[1][0].dtype == torch.bfloat16),
                   g2=part[2][0], c2=part[2][1], g2_is_bf16=int(part[2][0] is not None and part[2][0].dtype == torch.bfloat16),
                   n_src=len(src[i:i + 3]), out=dst, batch=B, seq=S, d_model=d)
            if not first:
                out += dst
            first = False
        return out, None, None


class _LayerNorm(torch.autograd.Function):
    """Row LayerNorm through nlh_layer_norm_forward / _backward. mode 0: fp32 output, 1: bf16
    output, 2: both (fp32 for the pooled levels, bf16 for the GEMM that follows)."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps, mode, grads=None, fan=None):
        """grads = (g_gamma, g_beta): buffers the backward accumulates the two parameter gradients
        into (the kernel adds with atomics); it then returns none for them. fan (dict or None):
        the block's gradient fan-in; the backward adds fan["r_dx"] (the gradient of x collected by
        the block's other consumers) to d_x inside the kernel."""
        ctx.grads = grads
        ctx.fan = fan
        x = x.contiguous()
        d = x.shape[-1]
        n = x.numel() // d
        dev = x.device
        o32 = torch.empty_like(x) if mode in (0, 2) else None
        o16 = torch.empty(x.shape, dtype=torch.bfloat16, device=dev) if mode in (1, 2) else None
        mean = torch.empty(n, dtype=torch.float32, device=dev)
        rstd = torch.empty(n, dtype=torch.float32, device=dev)
        D.call("nlh_layer_norm_forward", x=x, gamma=gamma.contiguous(), beta=beta.contiguous(),
               out_f32=o32, out_bf16=o16, mean_cache=mean, rstd_cache=rstd, n=n, d=d, eps=eps)
        ctx.save_for_backward(x, gamma, mean, rstd)
        ctx.mode = mode
        return o32 if mode == 0 else o16 if mode == 1 else (o32, o16)

    @staticmethod
    def backward(ctx, *grads):
        x, gamma, mean, rstd = ctx.saved_tensors
        d = x.shape[-1]
        n = x.numel() // d
        g32 = g16 = None
        for g in grads:
            if g is None:
                continue
            if g.dtype == torch.bfloat16:
                g16 = g.contiguous()
            else:
                g32 = g.contiguous()
        d_x = torch.empty_like(x)
        add_in = ctx.fan.pop("r_dx", None) if ctx.fan is not None else None
        if add_in is not None:
            assert ctx.grads is not None and (g32 is not None or g16 is not None)
            D.call("nlh_layer_norm_backward_fused", d_out_f32=g32, d_out_bf16=g16, g0=None, c0=1,
                   g0_is_bf16=0, g1=None, c1=1, g1_is_bf16=0, g2=None, c2=1, g2_is_bf16=0, n_src=0, seq=1,
                   x=x, res=None, res_is_bf16=0, add_in=add_in, gamma=gamma.contiguous(), mean_cache=mean,
                   rstd_cache=rstd, d_x=d_x, d_x_bf16=None, add_in_bf16=None, d_gamma=ctx.grads[0],
                   d_beta=ctx.grads[1], n=n, d=d)
            return d_x, None, None, None, None, None, None
        if ctx.grads is not None:
            if g32 is None and g16 is None:
                return d_x.zero_(), None, None, None, None, None, None
            D.call("nlh_layer_norm_backward", d_out_f32=g32, d_out_bf16=g16, x=x, gamma=gamma.contiguous(),
                   mean_cache=mean, rstd_cache=rstd, d_x=d_x, d_gamma=ctx.grads[0], d_beta=ctx.grads[1],
                   n=n, d=d)
            return d_x, None, None, None, None, None, None
        d_gb = torch.zeros(2, d, dtype=torch.float32, device=x.device)
        if g32 is None and g16 is None:
            return d_x.zero_(), d_gb[0], d_gb[1], None, None, None, None
        D.call("nlh_layer_norm_backward", d_out_f32=g32, d_out_bf16=g16, x=x, gamma=gamma.contiguous(),
               mean_cache=mean, rstd_cache=rstd, d_x=d_x, d_gamma=d_gb[0], d_beta=d_gb[1], n=n, d=d)
        return d_x, d_gb[0], d_gb[1], None, None, None, None


class _LayerNormPools(torch.autograd.Function):
    """LayerNorm of x [B, S, d] followed by the mean pools that feed the coarser CMS levels: returns
    the LayerNorm output (bf16 when out_bf16, the GEMM operand of level 0) and one mean-pooled copy
    per pool factor (ascending; coarser ones reduced from the finer one's sums when divisible).
    The backward is ONE kernel (nlh_layer_norm_backward_pooled): the pooled levels' gradients are
    upsampled and summed inside the LayerNorm backward instead of being written out first.
    grads = (g_gamma, g_beta): buffers the parameter gradients are accumulated into."""

    @staticmethod
    def forward(ctx, x, res, gamma, beta, eps, pools, out_bf16, grads, fan=None):
        """res (bf16 [B, S, d] or None): second addend of the LayerNorm input — the block's
        residual add x + attn_proj happens inside the LayerNorm kernels (forward and backward), the
        sum is never written. fan (dict or None, needs res): the block's gradient fan-in; the
        backward adds fan["c_dx"] / fan["c_dap"] (left by the MAG combine's backward) to the
        gradients of x / res inside the kernel, leaves the gradient of x in fan["r_dx"] for the
        attention LayerNorm's backward and returns none for x."""
        x = x.contiguous()
        B, S, d = x.shape
        n, dev = B * S, x.device
        o32 = torch.empty_like(x)
        o16 = torch.empty(x.shape, dtype=torch.bfloat16, device=dev) if out_bf16 else None
        mean = torch.empty(n, dtype=torch.float32, device=dev)
        rstd = torch.empty(n, dtype=torch.float32, device=dev)
        if res is not None:
            res = res.contiguous()
            assert res.dtype == torch.bfloat16
            D.call("nlh_layer_norm_residual_forward", x=x, res=res, res_is_bf16=1, gamma=gamma.contiguous(),
                   beta=beta.contiguous(), out_f32=o32, out_bf16=o16, mean_cache=mean, rstd_cache=rstd,
                   n=n, d=d, eps=eps)
        else:
            D.call("nlh_layer_norm_forward", x=x, gamma=gamma.contiguous(), beta=beta.contiguous(),
                   out_f32=o32, out_bf16=o16, mean_cache=mean, rstd_cache=rstd, n=n, d=d, eps=eps)
        dt = torch.bfloat16 if out_bf16 else torch.float32
        outs, prev = [], None                       # prev = (pool factor, unscaled sums)
        for i, c in enumerate(pools):
            later = any(c2 % c == 0 for c2 in pools[i + 1:])
            out = torch.empty(B, S // c, d, dtype=dt, device=dev)
            sums = torch.empty(B, S // c, d, dtype=torch.float32, device=dev) if later else None
            src, f = (prev[1], c // prev[0]) if prev is not None and c % prev[0] == 0 else (o32, c)
            D.call("nlh_mean_pool", src=src, factor=f, scale=1.0 / c, out=out, out_is_bf16=int(out_bf16),
                   sum_out=sums, rows_out=B * (S // c), d_model=d)
            if sums is not None:
                prev = (c, sums)
            outs.append(out)
        ctx.has_res = res is not None
        ctx.save_for_backward(x, gamma, mean, rstd, *([res] if res is not None else []))
        ctx.meta = (B, S, d, tuple(pools))
        ctx.grads = grads
        ctx.fan = fan if res is not None else None
        return (o16 if out_bf16 else o32, *outs)

    @staticmethod
    def backward(ctx, g_main, *gp):
        x, gamma, mean, rstd, *rest = ctx.saved_tensors
        res = rest[0] if ctx.has_res else None
        B, S, d, pools = ctx.meta
        src = [(g.contiguous(), c) for g, c in zip(gp, pools) if g is not None]
        assert len(src) <= 3, "at most three pooled levels"
        d_x = torch.empty_like(x)
        if res is not None:
            assert g_main is not None or src
            g32 = g16 = None
            if g_main is not None:
                g_main = g_main.contiguous()
                g16, g32 = (g_main, None) if g_main.dtype == torch.bfloat16 else (None, g_main)
            src = src + [(None, 1)] * (3 - len(src))
            isb = lambda t: int(t is not None and t.dtype == torch.bfloat16)
            fan = ctx.fan
            add_in = fan.pop("c_dx", None) if fan is not None else None
            add_bf = fan.pop("c_dap", None) if fan is not None else None
            d_res = torch.empty_like(res)
            D.call("nlh_layer_norm_backward_fused", d_out_f32=g32, d_out_bf16=g16,
                   g0=src[0][0], c0=src[0][1], g0_is_bf16=isb(src[0][0]),
                   g1=src[1][0], c1=src[1][1], g1_is_bf16=isb(src[1][0]),
                   g2=src[2][0], c2=src[2][1], g2_is_bf16=isb(src[2][0]),
                   n_src=sum(1 for g, _ in src if g is not None), seq=S, x=x, res=res, res_is_bf16=1,
                   add_in=add_in, gamma=gamma.contiguous(), mean_cache=mean, rstd_cache=rstd, d_x=d_x,
                   d_x_bf16=d_res, add_in_bf16=add_bf, d_gamma=ctx.grads[0], d_beta=ctx.grads[1],
                   n=B * S, d=d)
            if fan is not None:
                fan["r_dx"] = d_x
                return None, d_res, None, None, None, None, None, None, None
            return d_x, d_res, None, None, None, None, None, None, None
        if g_main is None and not src:
            return d_x.zero_(), None, None, None, None, None, None, None, None
        g32 = g16 = None
        if g_main is not None:
            g_main = g_main.contiguous()
            g16, g32 = (g_main, None) if g_main.dtype == torch.bfloat16 else (None, g_main)
        src = src + [(None, 1)] * (3 - len(src))
        isb = lambda t: int(t is not None and t.dtype == torch.bfloat16)
        D.call("nlh_layer_norm_backward_pooled", d_out_f32=g32, d_out_bf16=g16,
               g0=src[0][0], c0=src[0][1], g0_is_bf16=isb(src[0][0]),
               g1=src[1][0], c1=src[1][1], g1_is_bf16=isb(src[1][0]),
               g2=src[2][0], c2=src[2][1], g2_is_bf16=isb(src[2][0]),
               n_src=sum(1 for g, _ in src if g is not None), seq=S, x=x, gamma=gamma.contiguous(),
               mean_cache=mean, rstd_cache=rstd, d_x=d_x, d_gamma=ctx.grads[0], d_beta=ctx.grads[1],
               n=B * S, d=d)
        return d_x, None, None, None, None, None, None, None, None


class _CrossEntropy(torch.autograd.Function):
    """Mean cross-entropy over valid targets on fp32 or bf16 logits [n, vocab]
    (nlh_cross_entropy_forward / _backward). The backward overwrites the logits with their
    gradient, so the logits must not be used again after the loss."""

    @staticmethod
    def forward(ctx, logits, targets):
        n, vocab = logits.shape
        dev = logits.device
        acc = torch.zeros(2, dtype=torch.float32, device=dev)          # loss sum | (int) valid count
        cnt = acc[1:2].view(torch.int32)
        lse = torch.empty(n, dtype=torch.float32, device=dev)
        is_bf16 = int(logits.dtype == torch.bfloat16)
        D.call("nlh_cross_entropy_forward", logits=logits, logits_is_bf16=is_bf16, target_ids=targets,
               loss_sum=acc[0:1], lse=lse, valid_count=cnt, n=n, vocab=vocab)
        inv = 1.0 / cnt.float().clamp_min(1.0)
        ctx.save_for_backward(logits, targets, lse, inv)
        ctx.meta = (n, vocab, is_bf16)
        return (acc[0:1] * inv).reshape(())

    @staticmethod
    def backward(ctx, g):
        logits, targets, lse, inv = ctx.saved_tensors
        n, vocab, is_bf16 = ctx.meta
        scale = (g.float().reshape(1) * inv).contiguous()
        D.call("nlh_cross_entropy_backward", logits=logits, logits_is_bf16=is_bf16, target_ids=targets,
               lse=lse, grad_scale=scale, d_logits=logits, n=n, vocab=vocab, inv_count=1.0)
        return logits, None


class _Linear(torch.autograd.Function):
    """y = x W^T (or x W when transposed) on bf16 tensor cores, with the weight's bf16 copy taken
    from the model's per-step shadow arena (one cast of the whole arena per forward instead of one
    per weight) and the weight gradient added straight into the weight's slice of the fp32
    gradient arena (no per-weight cast and accumulation kernels). w itself is an input only so
    that the tape records the Function; no gradient is returned for it."""

    @staticmethod
    def forward(ctx, x, w, w16, grad_view, transposed, fp32_acc=True):
        x16 = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        y = torch.matmul(x16, w16) if transposed else F.linear(x16, w16)
        ctx.save_for_backward(x16, w16)
        ctx.grad_view, ctx.transposed, ctx.x_dtype, ctx.fp32_acc = grad_view, transposed, x.dtype, fp32_acc
        return y

    @staticmethod
    def backward(ctx, dy):
        x16, w16 = ctx.saved_tensors
        dy16 = dy if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16)
        dy2, x2 = dy16.reshape(-1, dy16.shape[-1]), x16.reshape(-1, x16.shape[-1])
        gv = ctx.grad_view
        # bf16 operands, fp32 accumulation and output, beta = 1 epilogue: grad += dW in one GEMM
        a, b = (x2.t(), dy2) if ctx.transposed else (dy2.t(), x2)
        dx = torch.matmul(dy16, w16.t() if ctx.transposed else w16)
        if ctx.fp32_acc:
            torch.addmm(gv, a, b, out_dtype=torch.float32, out=gv)
        else:
            gv.add_(torch.matmul(a, b))
        return (dx if ctx.x_dtype == torch.bfloat16 else dx.to(ctx.x_dtype)), None, None, None, None, None


class _Embedding(torch.autograd.Function):
    """x[t] = w_embed[ids[t]] through embedding_gather_cuda; the backward scatter-adds the output
    gradient straight into grad_out (the embedding's slice of the gradient arena,
    embedding_scatter_add_cuda), so no dense [vocab, d] temporary and no accumulation pass exist.
    Because of that side effect the Function returns no gradient for w_embed itself (w_embed is
    an input only so that the tape records the Function)."""

    @staticmethod
    def forward(ctx, ids, w_embed, grad_out):
        B, S = ids.shape
        d = w_embed.shape[1]
        ids32 = ids.reshape(-1).to(torch.int32).contiguous()
        out = torch.empty(B * S, d, dtype=torch.float32, device=w_embed.device)
        D.call("embedding_gather_cuda", w_embed=w_embed, input_ids=ids32, output=out, seq_len=B * S, d=d)
        ctx.save_for_backward(ids32)
        ctx.grad_out = grad_out
        ctx.mark_non_differentiable(ids32)
        return out.view(B, S, d)

    @staticmethod
    def backward(ctx, d_x):
        (ids32,) = ctx.saved_tensors
        d_x = d_x.contiguous().float()
        D.call("embedding_scatter_add_cuda", d_embedded=d_x.view(-1, d_x.shape[-1]), input_ids=ids32,
               d_embed=ctx.grad_out, seq_len=ids32.numel(), d=d_x.shape[-1])
        return None, None, None


def titans_memory(k, v, q, alpha, theta, eta, m0, chunk, slot=0, carry=None, ckpt=0):
    return _TitansMemory.apply(k, v, q, alpha, theta, eta, m0, chunk, slot, carry, ckpt)


def swa(q, k, v, num_heads, head_dim, window):
    return _SWA.apply(q, k, v, num_heads, head_dim, window)


class StackedMAG:
    """Parameters live in one flat fp32 arena (FlatAdamW); tensors below are views into it."""

    def __init__(self, cfg: StackedMAGConfig, batch_per_rank: int, device="cuda", seed=42,
                 memory_fn=titans_memory, swa_fn=swa):
        self.cfg, self.device = cfg, torch.device(device)
        self.memory_fn, self.swa_fn = memory_fn, swa_fn
        d, v, k = cfg.d_model, cfg.vocab, cfg.k
        names, shapes, clamp, level_of = [], [], {}, []

        def add(name, shape, level=None):
            names.append(name); shapes.append(shape); level_of.append(level)
            return len(names) - 1

        add("w_embed", (v, d)); add("w_unembed", (d, v))
        add("ln_final_gamma", (d,)); add("ln_final_beta", (d,))
        for b in range(cfg.n_blocks):
            p = f"b{b}."
            add(p + "w_qkv", (3 * d, d)); add(p + "w_o", (d, d))
            add(p + "ln_attn_gamma", (d,)); add(p + "ln_attn_beta", (d,))
            add(p + "ln_mem_gamma", (d,)); add(p + "ln_mem_beta", (d,))
            add(p + "alpha_mem", (k,))
            for l in range(k):
                q_ = p + f"l{l}."
                add(q_ + "w_kvq_mem", (3 * d, d), l)
                add(q_ + "w_gates", (3, 2 * d), l)        # rows: alpha, theta, eta
                add(q_ + "b_alpha", (1,), l)
                i = add(q_ + "b_theta", (1,), l)
                clamp[i] = (-10.0, 2.0)                    # gpu_stacked_optimizer.rs:667-671
                add(q_ + "b_eta", (1,), l)
        self.names, self.shapes, self.level_of = names, shapes, level_of
        self.opt = FlatAdamW([math.prod(s) for s in shapes], device=device, beta1=cfg.beta1,
                             beta2=cfg.beta2, eps=cfg.eps, weight_decay=cfg.weight_decay,
                             clamp=clamp)
        self.p, self.g = {}, {}
        for i, (n, s) in enumerate(zip(names, shapes)):
            w = self.opt.view(self.opt.w, i).view(s)
            w.requires_grad_(True)
            w.grad = self.opt.view(self.opt.g, i).view(s)
            self.p[n], self.g[n] = w, w.grad
        self._init(seed)
        # bf16 shadow of the parameter arena (GEMM operands), refreshed at the start of every forward
        import os
        self._use_linear = os.environ.get("NLH_MODEL_LINEAR", "1") == "1"
        self._use_embed = os.environ.get("NLH_MODEL_EMBED", "1") == "1"
        self._linear_fp32_acc = os.environ.get("NLH_MODEL_LINEAR_FP32", "1") == "1"
        self._w16, self.p16 = None, {}
        if cfg.bf16 and self.device.type == "cuda" and self._use_linear:
            self._w16 = torch.empty_like(self.opt.w, dtype=torch.bfloat16)
            for i, (n, sh) in enumerate(zip(names, shapes)):
                self.p16[n] = self.opt.view(self._w16, i).view(sh)
        # carried memory: one slot per (block, level, local sequence, head)
        nh, hd = cfg.num_heads, cfg.head_dim
        self.context = [[torch.zeros(batch_per_rank * nh, hd * hd, device=self.device)
                         for _ in range(k)] for _ in range(cfg.n_blocks)]
        self.global_step = 0
        self.level_steps = [0] * k

    @torch.no_grad()
    def _init(self, seed):
        """Seeded initialisation of the reference, draw for draw: StackedMAGParams::init and
        BlockParams::init (core/src/stacked_model.rs:69-119,172-208) with
        MemoryLevelParams::init_with_depth (core/src/model.rs:462-499). One xorshift64 stream
        (SimpleRng) per scope: `seed` for the embedding and unembedding, seed + 10000 (b + 1) for
        block b's attention projections, that + 1000 + 500 l for its level l."""
        import ctypes as C
        import numpy as np
        from . import ffi
        cfg = self.cfg
        d, v, nb = cfg.d_model, cfg.vocab, cfg.n_blocks
        lib = ffi.lib()

        class Stream:
            def __init__(self, sd):
                self.state = C.c_uint64(max(int(sd) & 0xFFFFFFFFFFFFFFFF, 1))

            def fill(self, dst, scale):
                buf = np.empty(dst.numel(), dtype=np.float32)
                lib.nlh_simple_rng_fill(C.byref(self.state), C.c_float(scale),
                                        buf.ctypes.data_as(C.c_void_p), C.c_int64(buf.size))
                dst.copy_(torch.from_numpy(buf).view(dst.shape))

        p = self.p
        proj = math.sqrt(2.0 / (d + d))
        depth = 1.0 / math.sqrt(2.0 * nb)              # GPT-2 depth scaling of output projections
        gate = math.sqrt(1.0 / (2 * d))
        emb = math.sqrt(1.0 / d)
        rng = Stream(seed)
        rng.fill(p["w_embed"], emb)
        rng.fill(p["w_unembed"], emb)
        p["ln_final_gamma"].fill_(1.0); p["ln_final_beta"].zero_()
        for b in range(nb):
            pre = f"b{b}."
            bseed = seed + 10_000 + b * 10_000
            brng = Stream(bseed)
            w_qkv = p[pre + "w_qkv"]
            for i in range(3):                          # w_q, w_k, w_v in the packed [q; k; v] rows
                brng.fill(w_qkv[i * d:(i + 1) * d], proj)
            brng.fill(p[pre + "w_o"], proj * depth)
            for n in ("ln_attn_", "ln_mem_"):
                p[pre + n + "gamma"].fill_(1.0); p[pre + n + "beta"].zero_()
            p[pre + "alpha_mem"].zero_()
            for l in range(cfg.k):
                q_ = pre + f"l{l}."
                lrng = Stream(bseed + 1000 + l * 500)
                w_kvq = p[q_ + "w_kvq_mem"]
                for i in range(3):                      # w_k_mem, w_v_mem, w_q_mem
                    lrng.fill(w_kvq[i * d:(i + 1) * d], proj * depth)
                for i in range(3):                      # w_alpha, w_theta, w_eta
                    lrng.fill(p[q_ + "w_gates"][i], gate)
                p[q_ + "b_alpha"].fill_(B_ALPHA[l]); p[q_ + "b_theta"].fill_(B_THETA[l]); p[q_ + "b_eta"].fill_(B_ETA[l])
        if cfg.tie_embeddings:
            self.p["w_embed"].copy_(self.p["w_unembed"].t())

    # ── forward ────────────────────────────────────────────────────────────
    def _mm(self, x, name, transposed=False):
        """x [.., in] times W^T (W = parameter `name`, [out, in]; transposed: x times W, W [in, out]).
        bf16 tensor-core GEMM when cfg.bf16: on the GPU through _Linear (shadow bf16 weights, weight
        gradient straight into the arena), else plain PyTorch operators."""
        w = self.p[name]
        if self.cfg.bf16 and x.is_cuda and self._w16 is not None and self._use_linear:
            return _Linear.apply(x, w, self.p16[name], self.g[name], transposed, self._linear_fp32_acc)
        if self.cfg.bf16:
            w16 = w.to(torch.bfloat16)
            return torch.matmul(x.to(torch.bfloat16), w16) if transposed else F.linear(x.to(torch.bfloat16), w16)
        return torch.matmul(x.float(), w) if transposed else F.linear(x.float(), w)

    def _refresh_shadow(self):
        """bf16 copy of the whole parameter arena for this forward (one kernel)."""
        if self._w16 is not None:
            with torch.no_grad():
                self._w16.copy_(self.opt.w)

    def _level(self, b, l, m_in):
        cfg, p = self.cfg, self.p
        B, S, d = m_in.shape
        nh, hd = cfg.num_heads, cfg.head_dim
        c = min(cfg.chunk_sizes[l], S)
        assert S % c == 0, "seq_len must be a multiple of every chunk size"
        sf = S // c
        x = m_in.view(B, sf, c, d).mean(2) if c > 1 else m_in
        pre = f"b{b}.l{l}."
        kvq = self._mm(x, pre + "w_kvq_mem").float()
        k, v, q = kvq.split(d, dim=-1)
        k = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-8)
        q = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-8)
        pre_g = torch.cat([k, v], dim=-1) @ p[pre + "w_gates"].t()
        alpha = torch.sigmoid(pre_g[..., 0] + p[pre + "b_alpha"])
        theta = F.softplus(pre_g[..., 1] + p[pre + "b_theta"])
        eta = torch.sigmoid(pre_g[..., 2] + p[pre + "b_eta"])
        heads = lambda t: t.reshape(B, sf, nh, hd).permute(0, 2, 1, 3).reshape(B * nh, sf, hd).contiguous()
        bro = lambda t: t.unsqueeze(1).expand(B, nh, sf).reshape(B * nh, sf).contiguous()
        chunk = 0 if l in cfg.exact_levels else min(cfg.chunk_sizes[l], sf)
        y, m_final = self.memory_fn(heads(k), heads(v), heads(q), bro(alpha), bro(theta), bro(eta),
                                    self.context[b][l], chunk)
        self.context[b][l].copy_(m_final.detach())
        y = y.view(B, nh, sf, hd).permute(0, 2, 1, 3).reshape(B, sf, d)
        return y.repeat_interleave(c, dim=1) if c > 1 else y

    def _level_fused(self, b, l, x, slot=0):
        """Level through the fused wrapper kernels; x is the level's (already pooled) input
        [B, S/c, d]. Returns the per-head output. slot: scratch slot of the library calls (a
        level that runs on a side stream must not share scratch with the other streams)."""
        cfg, p = self.cfg, self.p
        sf = x.shape[1]
        pre = f"b{b}.l{l}."
        kvq = self._mm(x, pre + "w_kvq_mem")
        g = self.g
        k, v, q, alpha, theta, eta = _LevelPrep.apply(
            kvq, p[pre + "w_gates"], p[pre + "b_alpha"], p[pre + "b_theta"], p[pre + "b_eta"],
            cfg.num_heads, slot,
            (g[pre + "w_gates"], g[pre + "b_alpha"], g[pre + "b_theta"], g[pre + "b_eta"]))
        chunk = 0 if l in cfg.exact_levels else min(cfg.chunk_sizes[l], sf)
        if self.memory_fn is titans_memory:   # carried memory updated in place by the Function
            y, _ = titans_memory(k, v, q, alpha, theta, eta, self.context[b][l], chunk, slot,
                                 self.context[b][l], cfg.exact_checkpoint if chunk == 0 else 0)
        else:
            y, m_final = self.memory_fn(k, v, q, alpha, theta, eta, self.context[b][l], chunk)
            self.context[b][l].copy_(m_final.detach())   # in place: addresses stay fixed for graph replay
        return y

    def _levels(self, b, inputs):
        """Outputs of all CMS levels of block b. With cfg.level_streams the levels >= 1 (short,
        latency-bound kernels) are issued on side streams and overlap level 0 on the GPU; the
        autograd engine replays the same stream assignment in the backward pass."""
        cfg = self.cfg
        if not cfg.level_streams or cfg.k < 2:
            return [self._level_fused(b, l, inputs[l]) for l in range(cfg.k)]
        main = torch.cuda.current_stream()
        if getattr(self, "_side", None) is None:
            self._side = [torch.cuda.Stream() for _ in range(cfg.k)]
        ys = [None] * cfg.k
        for l in range(1, cfg.k):
            st = self._side[l]
            st.wait_stream(main)
            with torch.cuda.stream(st):
                ys[l] = self._level_fused(b, l, inputs[l], slot=l)
            inputs[l].record_stream(st)
        ys[0] = self._level_fused(b, 0, inputs[0])
        for l in range(1, cfg.k):
            main.wait_stream(self._side[l])
            ys[l].record_stream(main)
        return ys

    def _ln(self, x, name, mode, fused, fan=None):
        p = self.p
        if fused:
            return _LayerNorm.apply(x, p[name + "gamma"], p[name + "beta"], 1e-5, mode,
                                    (self.g[name + "gamma"], self.g[name + "beta"]), fan)
        out = F.layer_norm(x, (x.shape[-1],), p[name + "gamma"], p[name + "beta"], 1e-5)
        return (out, out) if mode == 2 else out

    def forward(self, tokens, targets):
        cfg, p = self.cfg, self.p
        d, nh, hd = cfg.d_model, cfg.num_heads, cfg.head_dim
        fused = (cfg.fused_glue and tokens.is_cuda and cfg.k <= 4 and d <= 1024 and hd % 4 == 0)
        lp = 1 if (fused and cfg.bf16) else 0           # LayerNorm output feeding only a GEMM
        self._refresh_shadow()
        if fused and self._use_embed:
            x = _Embedding.apply(tokens, p["w_embed"], self.g["w_embed"])
        else:
            x = F.embedding(tokens, p["w_embed"])
        for b in range(cfg.n_blocks):
            pre = f"b{b}."
            self._mark_bucket(x, f"b{b}")            # fires once block b's backward has run
            S = x.shape[1]
            cs = [min(c, S) for c in cfg.chunk_sizes[:cfg.k]]
            uniq = sorted({c for c in cs if c > 1})
            # fan: the block's gradient fan-in. x and attn_proj both have three / two consumers in
            # the block; instead of autograd's sums (separate passes) the combine's backward hands
            # its contributions to the memory LayerNorm's backward, which hands the gradient of x to
            # the attention LayerNorm's backward; the kernels add them while they write.
            fan = {} if (fused and cfg.bf16 and d % 8 == 0 and len(uniq) <= 3) else None
            h = self._ln(x, pre + "ln_attn_", lp, fused, fan)
            qkv = self._mm(h, pre + "w_qkv")
            if cfg.bf16 or not qkv.is_cuda:
                qkv = qkv.to(torch.bfloat16)          # fp32 configurations keep fp32 attention on the GPU
            if fused and self.swa_fn is swa and qkv.dtype == torch.bfloat16:
                attn = _SWAPacked.apply(qkv, nh, hd, cfg.window)
            else:
                q, k, v = (t.contiguous() for t in qkv.split(d, dim=-1))
                attn = self.swa_fn(q, k, v, nh, hd, cfg.window)
            attn_raw = self._mm(attn, pre + "w_o")
            res1 = x + attn_raw if fan is None else None
            if fused:
                with torch.no_grad():
                    wts = torch.softmax(p[pre + "alpha_mem"], dim=0)
            else:
                wts = torch.softmax(p[pre + "alpha_mem"], dim=0)
            if fused:
                for c in cs:
                    assert S % c == 0, "seq_len must be a multiple of every chunk size"
                if fan is not None:                     # residual add, LayerNorm, pools and fan-in
                    m16, *pl = _LayerNormPools.apply(
                        x, attn_raw, p[pre + "ln_mem_gamma"], p[pre + "ln_mem_beta"], 1e-5, tuple(uniq), True,
                        (self.g[pre + "ln_mem_gamma"], self.g[pre + "ln_mem_beta"]), fan)
                    pooled = dict(zip(uniq, pl))
                elif d % 8 == 0 and len(uniq) <= 3:     # LayerNorm + pools, one backward kernel
                    m16, *pl = _LayerNormPools.apply(
                        res1, None, p[pre + "ln_mem_gamma"], p[pre + "ln_mem_beta"], 1e-5, tuple(uniq), cfg.bf16,
                        (self.g[pre + "ln_mem_gamma"], self.g[pre + "ln_mem_beta"]))
                    pooled = dict(zip(uniq, pl))
                else:
                    m32, m16 = self._ln(res1, pre + "ln_mem_", 2, True) if cfg.bf16 else \
                        (self._ln(res1, pre + "ln_mem_", 0, True),) * 2
                    pooled = dict(zip(uniq, _PoolLevels.apply(m32, tuple(uniq), cfg.bf16))) if uniq else {}
                ys = self._levels(b, [pooled.get(cs[l], m16) for l in range(cfg.k)])
                pools = cs
                x = _MagCombine.apply(x, attn_raw, wts, tuple(pools), nh, self.g[pre + "alpha_mem"], fan, *ys)
            else:
                m_in = self._ln(res1, pre + "ln_mem_", 0, False)
                attn_proj = attn_raw.float()
                y = None
                for l in range(cfg.k):
                    yl = self._level(b, l, m_in) * wts[l]
                    y = yl if y is None else y + yl
                x = x + attn_proj * torch.sigmoid(y)
        self._mark_bucket(x, "tail")                 # unembedding and final LayerNorm
        x = self._ln(x, "ln_final_", lp, fused)
        logits = self._mm(x, "w_unembed", transposed=True)
        if fused:
            return _CrossEntropy.apply(logits.view(-1, cfg.vocab), targets.reshape(-1).to(torch.int32))
        return F.cross_entropy(logits.float().view(-1, cfg.vocab), targets.reshape(-1))

    # ── one training step ──────────────────────────────────────────────────
    def pulse(self):
        """Active CMS levels this step (core/src/conductor.rs:136-155)."""
        cfg = self.cfg
        return [self.global_step % cs == 0 or cfg.seq_len >= cs for cs in cfg.chunk_sizes]

    def forward_backward(self, tokens, targets, process_group=None, world=1):
        """Loss (mean over the local batch) and its gradients, accumulated into the arena.
        With world > 1 (and cfg.overlap_grad_sync) the gradients are also averaged over the
        ranks here: the arena is laid out in the order the backward completes it
        backwards (embedding | unembedding + final LayerNorm | block 0 | block 1 | ...), so each
        block's slice is all-reduced (average) as soon as that block's backward has been
        issued and the exchange runs under the backward of the blocks below it; the embedding's
        slice goes last. sync_gradients() is then a no-op for this step."""
        overlap = (world > 1 and self.cfg.overlap_grad_sync and torch.distributed.is_available()
                   and torch.distributed.is_initialized())
        self._sync_state = dict(pg=process_group, works=[], seen=set(), world=world,
                                avg=tokens.is_cuda) if overlap else None
        loss = self.forward(tokens, targets)
        loss.backward()
        if overlap:
            st = self._sync_state
            for name in self._bucket_order():         # whatever no hook has covered (the embedding)
                if name not in st["seen"]:
                    self._reduce_bucket(name)
            for w in st["works"]:
                w.wait()                               # on the GPU the compute stream waits, not the host
            if not st["avg"]:                          # backends without an averaging reduction
                self.opt.g.mul_(1.0 / world)
            self._last_buckets = sorted(st["seen"])
            self._sync_state = None
            self._grads_synced = True
        return loss.detach()

    # ── bucketed gradient exchange ─────────────────────────────────────────
    def _bucket_order(self):
        return ["tail"] + [f"b{b}" for b in reversed(range(self.cfg.n_blocks))] + ["embed"]

    def _bucket_range(self, name):
        """[start, end) of a bucket in the flat arenas."""
        off = {n: self.opt.slices[i][0] for i, n in enumerate(self.names)}
        nb = self.cfg.n_blocks
        if name == "embed":
            return 0, off["w_unembed"]
        if name == "tail":
            return off["w_unembed"], off["b0.w_qkv"]
        b = int(name[1:])
        return off[f"b{b}.w_qkv"], (off[f"b{b + 1}.w_qkv"] if b + 1 < nb else self.opt.arena_len)

    def _reduce_bucket(self, name):
        st = self._sync_state
        st["seen"].add(name)
        o0, o1 = self._bucket_range(name)
        op = torch.distributed.ReduceOp.AVG if st["avg"] else torch.distributed.ReduceOp.SUM
        st["works"].append(torch.distributed.all_reduce(self.opt.g[o0:o1], op=op, group=st["pg"],
                                                        async_op=True))

    def _mark_bucket(self, x, name):
        """Tensor hook on the activation that enters a block (or the final LayerNorm): autograd
        calls it when that activation's gradient is complete, i.e. after every backward node of
        the block has been issued — side-stream levels included, their results are joined into
        the compute stream before the block's first LayerNorm backward runs."""
        if getattr(self, "_sync_state", None) is None or not x.requires_grad:
            return
        x.register_hook(lambda g, name=name: self._reduce_bucket(name))

    def sync_gradients(self, process_group=None, world=1):
        """Data-parallel gradient exchange when forward_backward() has not already done it:
        ONE all-reduce(SUM) over the flat gradient arena, then divide by the world size
        (core/src/distributed.rs:121-150 does the same per tensor). Inner-loop state (carried
        memories) is rank-local and never communicated."""
        if getattr(self, "_grads_synced", False):
            self._grads_synced = False
            return
        if world > 1:
            torch.distributed.all_reduce(self.opt.g, group=process_group)
            self.opt.g.mul_(1.0 / world)

    def _host_schedule(self):
        """Host bookkeeping of one step: pulse, global and per-level step counts, descriptors."""
        cfg = self.cfg
        active = self.pulse()
        self.global_step += 1
        for l in range(cfg.k):
            if active[l]:
                self.level_steps[l] += 1
        steps = [self.global_step if lv is None else max(self.level_steps[lv], 1)
                 for lv in self.level_of]
        act = [True if lv is None else active[lv] for lv in self.level_of]
        self.opt.prepare(steps, act)

    def _device_update(self):
        cfg = self.cfg
        self.opt.launch(cfg.lr, cfg.max_grad_norm)
        if cfg.tie_embeddings:
            with torch.no_grad():   # gpu_stacked_sync_embed_weights: w_embed <- w_unembed^T
                self.p["w_embed"].copy_(self.p["w_unembed"].t())
        self.opt.g.zero_()

    def apply_update(self):
        """Global-norm clip + AdamW with per-level step counts and pulse gating, weight tying."""
        self._host_schedule()
        self._device_update()

    def step(self, tokens, targets, process_group=None, world=1):
        """forward + backward + gradient all-reduce + clip + AdamW. Returns the local loss."""
        loss = self.forward_backward(tokens, targets, process_group, world)
        self.sync_gradients(process_group, world)
        self.apply_update()
        return loss

    def step_graphed(self, tokens, targets, process_group=None, world=1):
        """Same as step(), replayed from one CUDA graph (forward, backward, gradient all-reduce,
        clip, AdamW, weight tying): removes the per-launch host cost, which dominates when the
        per-rank batch is small. The first call runs two eager steps (sizes every allocation and
        the library workspace) and captures; later calls copy the inputs into static buffers and
        replay. Shapes must not change between calls."""
        if getattr(self, "_graph", None) is None:
            self._static_tok = tokens.clone()
            self._static_tgt = targets.clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self.step(self._static_tok, self._static_tgt, process_group, world)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            torch.cuda.empty_cache()
            self._host_schedule()
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._static_loss = self.forward_backward(self._static_tok, self._static_tgt,
                                                          process_group, world)
                self.sync_gradients(process_group, world)
                self._device_update()
            self._graph.replay()            # capture records only: run the scheduled step now
            self._graph_done = torch.cuda.Event()
            self._graph_done.record()
            return self._static_loss
        self._static_tok.copy_(tokens, non_blocking=True)
        self._static_tgt.copy_(targets, non_blocking=True)
        self._graph_done.synchronize()      # the previous replay has consumed the descriptors
        self._host_schedule()
        self._graph.replay()
        self._graph_done.record()
        return self._static_loss

    def n_params(self):
        return sum(math.prod(s) for s in self.shapes)
