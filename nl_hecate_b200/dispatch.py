"""Host-side mirror of the reference's kernel dispatch layer for the hot path.

``*_dd`` functions take device tensors and call the C ABI directly; they are
the counterpart of the ``*_dd`` wrappers in core/src/dispatch.rs:2093-3404.
``*_dispatch`` functions take host (numpy) arrays, copy them to the device, run
the kernel and copy the results back, like the ``*_dispatch`` functions of
core/src/dispatch.rs:330-1213 (``cuda_titans_forward`` etc.).

PyTorch is used only to own device memory and the stream. Every entry raises
if the CUDA library is missing or records an error: there is no CPU path here.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import ffi

RULE_DELTA, RULE_TITANS, RULE_HEBBIAN = 0, 1, 2
_PROTOS = None


def _protos():
    global _PROTOS
    if _PROTOS is None:
        _PROTOS = ffi.parse_header()
    return _PROTOS


def bind_stream(stream: torch.cuda.Stream | None = None) -> None:
    """Point the library at a torch stream (default: torch's current stream)."""
    s = stream if stream is not None else torch.cuda.current_stream()
    ffi.lib().nlh_set_stream(C.c_void_p(s.cuda_stream))


def call(name: str, **kw):
    """Call a C-ABI entry by name with keyword arguments named as in include/nlh_ffi.h.

    Tensors are passed as device pointers (they must be contiguous CUDA tensors),
    None as NULL. Status-returning entries are checked; void entries are checked
    through the library's recorded status.
    """
    ret, argtypes, argnames = _protos()[name]
    missing = [a for a in argnames if a not in kw]
    extra = [a for a in kw if a not in argnames]
    if missing or extra:
        raise TypeError(f"{name}: missing {missing}, unexpected {extra}")
    args = []
    for an, at in zip(argnames, argtypes):
        v = kw[an]
        if at is C.c_void_p:
            if v is None:
                args.append(C.c_void_p(0))
            elif isinstance(v, torch.Tensor):
                if not v.is_cuda or not v.is_contiguous():
                    raise ValueError(f"{name}.{an}: need a contiguous CUDA tensor")
                args.append(C.c_void_p(v.data_ptr()))
            elif isinstance(v, int):
                args.append(C.c_void_p(v))
            else:
                args.append(v)
        else:
            args.append(at(v))
    fn = getattr(ffi.lib(), name)
    bind_stream()
    if ret is None:
        ffi.lib().nlh_clear_status()   # void entries report through the recorded status
    rc = fn(*args)
    if ret is C.c_int32:
        ffi.check(rc, name)
    elif ret is C.c_uint32:
        if rc != 0:
            raise RuntimeError(f"{name}: cudaError {rc}")
    elif ret is None:
        ffi.check_void(name)
    return rc


class workspace_slot:
    """Context manager: the library calls inside use scratch slot ``slot`` (launches that may
    overlap on the GPU, i.e. run on different streams, must not share a slot)."""

    def __init__(self, slot: int):
        self.slot = int(slot)

    def __enter__(self):
        if self.slot:
            ffi.check(ffi.lib().nlh_set_workspace_slot(self.slot), "nlh_set_workspace_slot")
        return self

    def __exit__(self, *exc):
        if self.slot:
            ffi.lib().nlh_set_workspace_slot(0)
        return False


def _f32(*shape, device):
    return torch.empty(*shape, dtype=torch.float32, device=device)


def checkpoint_count(seq_len: int, c: int) -> int:
    """Slots written by the checkpointed forwards (core/src/gpu_forward.rs:2885-2900)."""
    assert c > 0
    return 1 + sum(1 for t in range(seq_len) if (t + 1) % c == 0 or t + 1 == seq_len)


# ── memory rules, device tensors ───────────────────────────────────────────
# Shapes: k,v,q,d_y [N,S,d]; gates [N,S]; m0,s0 [N,d*d]; states [N,(S+1),d*d].

def _zero_grads(k, alpha, d, want_initial=True):
    """Backward outputs of a Titans entry: d_k, d_v, d_q like k and d_alpha, d_theta, d_eta like
    alpha are overwritten by every kernel path, so they are left uninitialised; d_m_initial and
    d_s_initial [d*d] are summed over the batch with atomics and start from zero (one small
    fill). want_initial=False passes NULL for those two: the entries then skip them."""
    dk, dv, dq = (torch.empty_like(k) for _ in range(3))
    da, dt, de = (torch.empty_like(alpha) for _ in range(3))
    if not want_initial:
        return dk, dv, dq, da, dt, de, None, None
    init = torch.zeros(2, d * d, dtype=torch.float32, device=k.device)
    return dk, dv, dq, da, dt, de, init[0], init[1]


def titans_forward_dd(k, v, q, alpha, theta, eta, m0, s0, error_clip=0.0, m_norm_max=0.0,
                      store_s=True):
    """store_s=False passes s_states = NULL: the momentum trajectory is not written (half the
    HBM traffic); titans_backward_dd(..., ss=None) then derives S_t from consecutive M states."""
    n, s, d = k.shape
    ms = _f32(n, s + 1, d * d, device=k.device)
    ss = _f32(n, s + 1, d * d, device=k.device) if store_s else None
    y = _f32(n, s, d, device=k.device)
    call("titans_forward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta, eta=eta,
         m_initial=m0, s_initial=s0, m_states=ms, s_states=ss, y=y, seq_len=s, d=d, batch_size=n,
         input_stride=s, m_stride=d * d, error_clip=error_clip, m_norm_max=m_norm_max)
    return ms, ss, y


def titans_backward_dd(k, v, q, alpha, theta, eta, ms, ss, d_y, error_clip=0.0, want_initial=True):
    n, s, d = k.shape
    dk, dv, dq, da, dt, de, dm0, ds0 = _zero_grads(k, alpha, d, want_initial)
    call("titans_backward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta, eta=eta,
         m_states=ms, s_states=ss, d_y=d_y, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da,
         d_theta=dt, d_eta=de, d_m_initial=dm0, d_s_initial=ds0, seq_len=s, d=d, batch_size=n,
         error_clip=error_clip)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dt, d_eta=de, d_m_initial=dm0,
                d_s_initial=ds0)


def mlp_state_size(d, d_hidden):
    """Floats in one packed MLP memory state: W1[d_hidden,d], b1[d_hidden], W2[d,d_hidden], b2[d]."""
    return d_hidden * d + d_hidden + d * d_hidden + d


def titans_mlp_forward_dd(k, v, q, alpha, theta, eta, m0, s0, d_hidden, activation=0, m_norm_max=0.0):
    """Titans LMM with a two-layer MLP memory (titans_mlp_forward_f32_cuda): m0, s0 [N, state];
    returns m_states, s_states [N, S+1, state] and y [N, S, d]."""
    n, s, d = k.shape
    ssz = mlp_state_size(d, d_hidden)
    ms = torch.empty(n, s + 1, ssz, dtype=torch.float32, device=k.device)
    ss = torch.empty(n, s + 1, ssz, dtype=torch.float32, device=k.device)
    y = torch.empty(n, s, d, dtype=torch.float32, device=k.device)
    call("titans_mlp_forward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta, eta=eta,
         m_initial=m0, s_initial=s0, m_states=ms, s_states=ss, y=y, seq_len=s, d=d, d_hidden=d_hidden,
         batch_size=n, input_stride=s * d, m_stride=(s + 1) * ssz, activation=activation,
         m_norm_max=m_norm_max)
    return ms, ss, y


def titans_mlp_backward_dd(k, v, q, alpha, theta, eta, ms, ss, d_y, d_hidden, activation=0):
    """Backward twin; d_m_initial / d_s_initial [state] are summed over the N problems."""
    n, s, d = k.shape
    ssz = mlp_state_size(d, d_hidden)
    dk, dv, dq = (torch.empty_like(k) for _ in range(3))
    da, dt, de = (torch.empty_like(alpha) for _ in range(3))
    dm0 = torch.zeros(ssz, dtype=torch.float32, device=k.device)
    ds0 = torch.zeros(ssz, dtype=torch.float32, device=k.device)
    call("titans_mlp_backward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta, eta=eta,
         m_states=ms, s_states=ss, d_y=d_y, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_theta=dt,
         d_eta=de, d_m_initial=dm0, d_s_initial=ds0, seq_len=s, d=d, d_hidden=d_hidden, batch_size=n,
         input_stride=s * d, m_stride=(s + 1) * ssz, activation=activation, m_norm_max=0.0)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dt, d_eta=de, d_m_initial=dm0, d_s_initial=ds0)


def delta_forward_dd(k, v, q, alpha, theta, m0, error_clip=0.0, m_norm_max=0.0, dgd=False):
    n, s, d = k.shape
    ms = _f32(n, s + 1, d * d, device=k.device)
    y = _f32(n, s, d, device=k.device)
    if dgd:
        call("dgd_forward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
             m_initial=m0, m_states=ms, y=y, seq_len=s, d=d, batch_size=n, input_stride=s,
             m_stride=d * d, error_clip=error_clip)
    else:
        call("delta_forward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
             m_initial=m0, m_states=ms, y=y, seq_len=s, d=d, batch_size=n, input_stride=s,
             m_stride=d * d, error_clip=error_clip, m_norm_max=m_norm_max)
    return ms, y


def delta_backward_dd(k, v, q, alpha, theta, ms, d_y, error_clip=0.0, dgd=False):
    n, s, d = k.shape
    dk, dv, dq = (torch.zeros_like(k) for _ in range(3))
    da, dt = (torch.zeros_like(alpha) for _ in range(2))
    dm0 = torch.zeros(d * d, dtype=torch.float32, device=k.device)
    if dgd:
        assert n == 1, "dgd_backward_f32_cuda has no batch argument"
        call("dgd_backward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
             m_states=ms, d_y=d_y, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_theta=dt,
             d_m_initial=dm0, seq_len=s, d=d, error_clip=error_clip)
    else:
        call("delta_backward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
             m_states=ms, d_y=d_y, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_theta=dt,
             d_m_initial=dm0, seq_len=s, d=d, batch_size=n, error_clip=error_clip)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dt, d_m_initial=dm0)


def hebbian_forward_dd(k, v, q, alpha, m0):
    n, s, d = k.shape
    ms = _f32(n, s + 1, d * d, device=k.device)
    y = _f32(n, s, d, device=k.device)
    call("hebbian_forward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, m_initial=m0,
         m_states=ms, y=y, seq_len=s, d=d, batch_size=n, input_stride=s, m_stride=d * d)
    return ms, y


def hebbian_backward_dd(k, v, q, alpha, ms, d_y):
    n, s, d = k.shape
    assert n == 1, "hebbian_backward_f32_cuda has no batch argument"
    dk, dv, dq = (torch.zeros_like(k) for _ in range(3))
    da = torch.zeros_like(alpha)
    dm0 = torch.zeros(d * d, dtype=torch.float32, device=k.device)
    call("hebbian_backward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, m_states=ms, d_y=d_y,
         d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_m_initial=dm0, seq_len=s, d=d)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_m_initial=dm0)


def titans_chunkwise_forward_dd(k, v, q, alpha, theta, eta, m0, s0, chunk, error_clip=0.0,
                                m_norm_max=0.0):
    n, s, d = k.shape
    nc = (s + chunk - 1) // chunk
    mc = _f32(n, nc + 1, d * d, device=k.device)
    sc = _f32(n, nc + 1, d * d, device=k.device)
    y = _f32(n, s, d, device=k.device)
    call("titans_chunkwise_forward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
         eta=eta, m_initial=m0, s_initial=s0, m_chunk_states=mc, s_chunk_states=sc, y=y,
         seq_len=s, d=d, batch_size=n, chunk_size=chunk, error_clip=error_clip,
         m_norm_max=m_norm_max)
    return mc, sc, y


def titans_chunkwise_backward_dd(k, v, q, alpha, theta, eta, mc, sc, d_y, chunk, error_clip=0.0,
                                 m_norm_max=0.0, want_initial=True):
    n, s, d = k.shape
    dk, dv, dq, da, dt, de, dm0, ds0 = _zero_grads(k, alpha, d, want_initial)
    call("titans_chunkwise_backward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
         eta=eta, m_chunk_states=mc, s_chunk_states=sc, d_y=d_y, d_k_mem=dk, d_v_mem=dv,
         d_q_mem=dq, d_alpha=da, d_theta=dt, d_eta=de, d_m_initial=dm0, d_s_initial=ds0,
         seq_len=s, d=d, batch_size=n, chunk_size=chunk, error_clip=error_clip,
         m_norm_max=m_norm_max)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dt, d_eta=de, d_m_initial=dm0,
                d_s_initial=ds0)


def delta_chunkwise_forward_dd(k, v, q, alpha, theta, m0, chunk, error_clip=0.0, m_norm_max=0.0):
    n, s, d = k.shape
    nc = (s + chunk - 1) // chunk
    mc = _f32(n, nc + 1, d * d, device=k.device)
    y = _f32(n, s, d, device=k.device)
    call("delta_chunkwise_forward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
         m_initial=m0, m_chunk_states=mc, y=y, seq_len=s, d=d, batch_size=n, chunk_size=chunk,
         error_clip=error_clip, m_norm_max=m_norm_max)
    return mc, y


def delta_chunkwise_backward_dd(k, v, q, alpha, theta, mc, d_y, chunk, error_clip=0.0,
                                m_norm_max=0.0):
    n, s, d = k.shape
    dk, dv, dq = (torch.zeros_like(k) for _ in range(3))
    da, dt = (torch.zeros_like(alpha) for _ in range(2))
    dm0 = torch.zeros(d * d, dtype=torch.float32, device=k.device)
    call("delta_chunkwise_backward_f32_cuda", k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
         m_chunk_states=mc, d_y=d_y, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da, d_theta=dt,
         d_m_initial=dm0, seq_len=s, d=d, batch_size=n, chunk_size=chunk, error_clip=error_clip,
         m_norm_max=m_norm_max)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dt, d_m_initial=dm0)


# ── recompute-style training pair (additive API) ───────────────────────────
def rule_forward(rule, k, v, q, alpha, theta, eta, m0, s0, interval, chunk=0, error_clip=0.0,
                 m_norm_max=0.0):
    n, s, d = k.shape
    slots = (s + interval - 1) // interval + 1
    mc = _f32(n, slots, d * d, device=k.device)
    sc = _f32(n, slots, d * d, device=k.device) if rule == RULE_TITANS else None
    y = _f32(n, s, d, device=k.device)
    call("nlh_rule_forward", rule=rule, k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
         eta=eta, m_initial=m0, s_initial=s0, m_ckpt=mc, s_ckpt=sc, y=y, seq_len=s, d=d,
         batch_size=n, interval=interval, chunk_size=chunk, error_clip=error_clip,
         m_norm_max=m_norm_max)
    return mc, sc, y


def rule_backward(rule, k, v, q, alpha, theta, eta, mc, sc, d_y, interval, chunk=0, error_clip=0.0,
                  m_norm_max=0.0):
    n, s, d = k.shape
    dk, dv, dq = (torch.empty_like(k) for _ in range(3))
    da = torch.empty_like(alpha)
    dt = torch.empty_like(alpha) if rule != RULE_HEBBIAN else None
    de = torch.empty_like(alpha) if rule == RULE_TITANS else None
    dm0 = _f32(n, d * d, device=k.device)
    ds0 = _f32(n, d * d, device=k.device) if rule == RULE_TITANS else None
    call("nlh_rule_backward", rule=rule, k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
         eta=eta, m_ckpt=mc, s_ckpt=sc, d_y=d_y, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da,
         d_theta=dt, d_eta=de, d_m_initial=dm0, d_s_initial=ds0, seq_len=s, d=d, batch_size=n,
         interval=interval, chunk_size=chunk, error_clip=error_clip, m_norm_max=m_norm_max)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dt, d_eta=de, d_m_initial=dm0,
                d_s_initial=ds0)


def titans_frozen_stream_forward(k, v, q, alpha, theta, eta, m0, s0, chunk):
    """Frozen-M0 chunkwise Titans forward that stores EVERY state (nlh_rule_forward with
    interval = 1): ms [N, S+1, d*d], no momentum trajectory. For short chunks, where the
    backward then streams the states instead of recomputing chunk windows."""
    n, s, d = k.shape
    ms = _f32(n, s + 1, d * d, device=k.device)
    y = _f32(n, s, d, device=k.device)
    call("nlh_rule_forward", rule=RULE_TITANS, k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
         eta=eta, m_initial=m0, s_initial=s0, m_ckpt=ms, s_ckpt=None, y=y, seq_len=s, d=d,
         batch_size=n, interval=1, chunk_size=chunk, error_clip=0.0, m_norm_max=0.0)
    return ms, y


def titans_frozen_stream_backward(k, v, q, alpha, theta, eta, ms, d_y, chunk, want_initial=True):
    """Backward twin (nlh_rule_backward with interval = 1). d_m_initial / d_s_initial are per
    problem [N, d*d]; want_initial=False passes NULL for both."""
    n, s, d = k.shape
    dk, dv, dq = (torch.empty_like(k) for _ in range(3))
    da, dt, de = (torch.empty_like(alpha) for _ in range(3))
    dm0 = _f32(n, d * d, device=k.device) if want_initial else None
    ds0 = _f32(n, d * d, device=k.device) if want_initial else None
    call("nlh_rule_backward", rule=RULE_TITANS, k_mem=k, v_mem=v, q_mem=q, alpha=alpha, theta=theta,
         eta=eta, m_ckpt=ms, s_ckpt=None, d_y=d_y, d_k_mem=dk, d_v_mem=dv, d_q_mem=dq, d_alpha=da,
         d_theta=dt, d_eta=de, d_m_initial=dm0, d_s_initial=ds0, seq_len=s, d=d, batch_size=n,
         interval=1, chunk_size=chunk, error_clip=0.0, m_norm_max=0.0)
    return dict(d_k=dk, d_v=dv, d_q=dq, d_alpha=da, d_theta=dt, d_eta=de, d_m_initial=dm0,
                d_s_initial=ds0)


# ── SWA ────────────────────────────────────────────────────────────────────
# q,k,v,out: [B,S,H*hd] bf16; attn_weights [B,H,S,n_p+W] bf16; grads f32.

def swa_forward_dd(q, k, v, num_heads, head_dim, window, n_persistent=0, want_weights=True):
    b, s, _ = q.shape
    out = torch.empty_like(q)
    aw = (torch.empty(b, num_heads, s, n_persistent + window, dtype=torch.bfloat16, device=q.device)
          if want_weights else None)
    call("swa_forward_f32_cuda", q=q, k=k, v=v, out=out, attn_weights=aw, seq_len=s,
         num_heads=num_heads, head_dim=head_dim, window_size=window, batch_size=b,
         n_persistent=n_persistent)
    return out, aw


def swa_backward_dd(q, k, v, aw, d_out, num_heads, head_dim, window, n_persistent=0):
    b, s, td = q.shape
    dq, dk, dv = (torch.zeros(b, s, td, dtype=torch.float32, device=q.device) for _ in range(3))
    call("swa_backward_f32_cuda", q=q, k=k, v=v, attn_weights=aw, d_attn_out=d_out, d_q=dq, d_k=dk,
         d_v=dv, seq_len=s, num_heads=num_heads, head_dim=head_dim, window_size=window,
         batch_size=b, n_persistent=n_persistent)
    return dq, dk, dv


def swa_forward_lse(q, k, v, num_heads, head_dim, window, n_persistent=0):
    b, s, _ = q.shape
    out = torch.empty_like(q)
    lse = _f32(b, num_heads, s, device=q.device)
    call("nlh_swa_forward", q=q, k=k, v=v, out=out, lse=lse, seq_len=s, num_heads=num_heads,
         head_dim=head_dim, window_size=window, batch_size=b, n_persistent=n_persistent)
    return out, lse


def swa_backward_lse(q, k, v, out, lse, d_out, num_heads, head_dim, window, n_persistent=0):
    b, s, td = q.shape
    dq, dk, dv = (torch.empty(b, s, td, dtype=torch.float32, device=q.device) for _ in range(3))
    call("nlh_swa_backward", q=q, k=k, v=v, out=out, lse=lse, d_attn_out=d_out, d_q=dq, d_k=dk,
         d_v=dv, seq_len=s, num_heads=num_heads, head_dim=head_dim, window_size=window,
         batch_size=b, n_persistent=n_persistent)
    return dq, dk, dv


def swa_forward_f32(q, k, v, num_heads, head_dim, window, n_persistent=0):
    """fp32 SWA (nlh_swa_forward_f32): q, k, v fp32 [B, S, H*hd]; returns (out fp32, lse)."""
    b, s, _ = q.shape
    out = torch.empty_like(q)
    lse = _f32(b, num_heads, s, device=q.device)
    call("nlh_swa_forward_f32", q=q, k=k, v=v, out=out, lse=lse, seq_len=s, num_heads=num_heads,
         head_dim=head_dim, window_size=window, batch_size=b, n_persistent=n_persistent)
    return out, lse


def swa_backward_f32(q, k, v, out, lse, d_out, num_heads, head_dim, window, n_persistent=0):
    b, s, td = q.shape
    dq, dk, dv = (torch.empty(b, s, td, dtype=torch.float32, device=q.device) for _ in range(3))
    call("nlh_swa_backward_f32", q=q, k=k, v=v, out=out, lse=lse, d_attn_out=d_out, d_q=dq, d_k=dk,
         d_v=dv, seq_len=s, num_heads=num_heads, head_dim=head_dim, window_size=window,
         batch_size=b, n_persistent=n_persistent)
    return dq, dk, dv


# ── AdamW ──────────────────────────────────────────────────────────────────
def adamw_update_dd(w, g, m, v, lr, beta1, beta2, eps, bc1_inv, bc2_inv, weight_decay):
    call("adamw_update_cuda", w=w, g=g, m=m, v=v, n=w.numel(), lr=lr, beta1=beta1, beta2=beta2,
         eps=eps, bc1_inv=bc1_inv, bc2_inv=bc2_inv, weight_decay=weight_decay)


def grad_norm_clip_dd(grads, max_norm):
    """Global-norm clip over a list of tensors with the reference's kernel sequence
    (core/src/gpu_stacked_optimizer.rs:193-345). Returns (norm, scale) as device scalars."""
    dev = grads[0].device
    total = sum((g.numel() + 255) // 256 for g in grads)
    partial = _f32(total, device=dev)
    off = 0
    nb = C.c_int32(0)
    for g in grads:
        call("grad_norm_sq_cuda", g=g, partial_sums=partial[off:], n=g.numel(),
             out_num_blocks=C.cast(C.pointer(nb), C.c_void_p))
        off += nb.value
    assert off == total
    norm, scale = _f32(1, device=dev), _f32(1, device=dev)
    call("reduce_partials_clip_cuda", partial_sums=partial, total_partials=total,
         max_grad_norm=max_norm, out_norm=norm, out_scale=scale)
    for g in grads:
        call("grad_scale_conditional_cuda", g=g, scale_ptr=scale, n=g.numel())
    return norm, scale


# ── host-slice API (H2D + kernel + D2H), numpy in / numpy out ───────────────
def _dev(a, dtype=torch.float32):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.to("cuda", non_blocking=False).to(dtype) if t.dtype != dtype else t.to("cuda")


def titans_forward_dispatch(k, v, q, alpha, theta, eta, m0, s0, error_clip=0.0, m_norm_max=0.0):
    """Counterpart of titans_forward_dispatch (core/src/dispatch.rs:810-839), batch = 1."""
    s, d = k.shape
    ms, ss, y = titans_forward_dd(_dev(k)[None], _dev(v)[None], _dev(q)[None], _dev(alpha)[None],
                                  _dev(theta)[None], _dev(eta)[None], _dev(m0)[None],
                                  _dev(s0)[None], error_clip, m_norm_max)
    return ms[0].cpu().numpy(), ss[0].cpu().numpy(), y[0].cpu().numpy()


# ── opaque-VJP registry over the C ABI (host slices, as on the reference's tape) ──
OPAQUE_KEYS = {"DeltaRule": 0, "TitansLMM": 1, "HebbianRule": 2, "DGD": 9, "SWA": 10,
               "FrozenDeltaRule": 11, "FrozenTitansLMM": 12, "FrozenHebbianRule": 13}


def opaque_backward(key, d_outputs, saved, in_lens):
    """Counterpart of an ``OpaqueBackwardFn`` (core/src/tape.rs:141-145): host float32 arrays in,
    list of host float32 input gradients out (lengths ``in_lens``). ``key`` is an OpaqueKey name
    or number; keys without a GPU adapter raise."""
    if isinstance(key, str):
        key = OPAQUE_KEYS[key]
    d_outputs = [np.ascontiguousarray(a, dtype=np.float32).ravel() for a in d_outputs]
    saved = [np.ascontiguousarray(a, dtype=np.float32).ravel() for a in saved]
    d_inputs = [np.zeros(int(n), dtype=np.float32) for n in in_lens]

    def pack(arrs):
        ptrs = (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])
        lens = (C.c_int64 * len(arrs))(*[a.size for a in arrs])
        return ptrs, lens

    po, lo = pack(d_outputs)
    ps, ls = pack(saved)
    pi, li = pack(d_inputs)
    call("nlh_opaque_backward", key=key, n_out=len(d_outputs), d_outputs=po, out_len=lo,
         n_saved=len(saved), saved=ps, saved_len=ls, n_in=len(d_inputs), d_inputs=pi, in_len=li)
    return d_inputs


# ── compiled host-slice dispatch layer (core/src/dispatch.rs `*_dispatch` functions) ──
def _h(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _hp(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def host_rule_forward(rule, k, v, q, alpha, theta=None, eta=None, m0=None, s0=None, error_clip=0.0,
                      m_norm_max=0.0):
    """Host arrays in, host arrays out through nlh_{delta,titans,hebbian,dgd}_forward_dispatch
    (one sequence: k,v,q [s, d]). Returns dict(m_states, y[, s_states])."""
    k, v, q, alpha, m0 = map(_h, (k, v, q, alpha, m0))
    s, d = k.shape
    ms, y = np.empty((s + 1, d * d), np.float32), np.empty((s, d), np.float32)
    out = {"m_states": ms, "y": y}
    if rule == "titans":
        theta, eta, s0 = map(_h, (theta, eta, s0))
        ss = np.empty((s + 1, d * d), np.float32)
        out["s_states"] = ss
        call("nlh_titans_forward_dispatch", k_mem=_hp(k), v_mem=_hp(v), q_mem=_hp(q), alpha=_hp(alpha),
             theta=_hp(theta), eta=_hp(eta), m_initial=_hp(m0), s_initial=_hp(s0), m_states=_hp(ms),
             s_states=_hp(ss), y=_hp(y), seq_len=s, d=d, error_clip=error_clip, m_norm_max=m_norm_max)
    elif rule == "hebbian":
        call("nlh_hebbian_forward_dispatch", k_mem=_hp(k), v_mem=_hp(v), q_mem=_hp(q), alpha=_hp(alpha),
             m_initial=_hp(m0), m_states=_hp(ms), y=_hp(y), seq_len=s, d=d)
    elif rule == "dgd":
        theta = _h(theta)
        call("nlh_dgd_forward_dispatch", k_mem=_hp(k), v_mem=_hp(v), q_mem=_hp(q), alpha=_hp(alpha),
             theta=_hp(theta), m_initial=_hp(m0), m_states=_hp(ms), y=_hp(y), seq_len=s, d=d,
             error_clip=error_clip)
    else:
        theta = _h(theta)
        call("nlh_delta_forward_dispatch", k_mem=_hp(k), v_mem=_hp(v), q_mem=_hp(q), alpha=_hp(alpha),
             theta=_hp(theta), m_initial=_hp(m0), m_states=_hp(ms), y=_hp(y), seq_len=s, d=d,
             error_clip=error_clip, m_norm_max=m_norm_max)
    return out


def host_rule_backward(rule, k, v, q, alpha, m_states, d_y, theta=None, eta=None, s_states=None,
                       error_clip=0.0):
    k, v, q, alpha, m_states, d_y = map(_h, (k, v, q, alpha, m_states, d_y))
    s, d = k.shape
    z = lambda *sh: np.zeros(sh, np.float32)
    g = {"d_k": z(s, d), "d_v": z(s, d), "d_q": z(s, d), "d_alpha": z(s), "d_m_initial": z(d * d)}
    common = dict(k_mem=_hp(k), v_mem=_hp(v), q_mem=_hp(q), alpha=_hp(alpha), m_states=_hp(m_states),
                  d_y=_hp(d_y), d_k_mem=_hp(g["d_k"]), d_v_mem=_hp(g["d_v"]), d_q_mem=_hp(g["d_q"]),
                  d_alpha=_hp(g["d_alpha"]), d_m_initial=_hp(g["d_m_initial"]), seq_len=s, d=d)
    if rule == "hebbian":
        call("nlh_hebbian_backward_dispatch", **common)
        return g
    theta = _h(theta)
    g["d_theta"] = z(s)
    common.update(theta=_hp(theta), d_theta=_hp(g["d_theta"]), error_clip=error_clip)
    if rule == "titans":
        eta, s_states = _h(eta), _h(s_states)
        g["d_eta"], g["d_s_initial"] = z(s), z(d * d)
        call("nlh_titans_backward_dispatch", eta=_hp(eta), s_states=_hp(s_states), d_eta=_hp(g["d_eta"]),
             d_s_initial=_hp(g["d_s_initial"]), **common)
    else:
        call("nlh_dgd_backward_dispatch" if rule == "dgd" else "nlh_delta_backward_dispatch", **common)
    return g


def host_titans_mlp_pair(k, v, q, alpha, theta, eta, m0, s0, d_y, d_hidden, activation=0, m_norm_max=0.0):
    """Host arrays in, host arrays out through nlh_titans_mlp_{forward,backward}_dispatch
    (k, v, q, d_y [n, s, d]; gates [n, s]; m0, s0 [n, state]). Returns (forward dict, gradient dict)."""
    k, v, q, alpha, theta, eta, m0, s0, d_y = map(_h, (k, v, q, alpha, theta, eta, m0, s0, d_y))
    n, s, d = k.shape
    ssz = mlp_state_size(d, d_hidden)
    f = {"m_states": np.empty((n, s + 1, ssz), np.float32), "s_states": np.empty((n, s + 1, ssz), np.float32),
         "y": np.empty((n, s, d), np.float32)}
    call("nlh_titans_mlp_forward_dispatch", k_mem=_hp(k), v_mem=_hp(v), q_mem=_hp(q), alpha=_hp(alpha),
         theta=_hp(theta), eta=_hp(eta), m_initial=_hp(m0), s_initial=_hp(s0), m_states=_hp(f["m_states"]),
         s_states=_hp(f["s_states"]), y=_hp(f["y"]), seq_len=s, d=d, d_hidden=d_hidden, batch_size=n,
         activation=activation, m_norm_max=m_norm_max)
    e = lambda *sh: np.empty(sh, np.float32)
    g = {"d_k": e(n, s, d), "d_v": e(n, s, d), "d_q": e(n, s, d), "d_alpha": e(n, s), "d_theta": e(n, s),
         "d_eta": e(n, s), "d_m_initial": e(ssz), "d_s_initial": e(ssz)}
    call("nlh_titans_mlp_backward_dispatch", k_mem=_hp(k), v_mem=_hp(v), q_mem=_hp(q), alpha=_hp(alpha),
         theta=_hp(theta), eta=_hp(eta), m_states=_hp(f["m_states"]), s_states=_hp(f["s_states"]), d_y=_hp(d_y),
         d_k_mem=_hp(g["d_k"]), d_v_mem=_hp(g["d_v"]), d_q_mem=_hp(g["d_q"]), d_alpha=_hp(g["d_alpha"]),
         d_theta=_hp(g["d_theta"]), d_eta=_hp(g["d_eta"]), d_m_initial=_hp(g["d_m_initial"]),
         d_s_initial=_hp(g["d_s_initial"]), seq_len=s, d=d, d_hidden=d_hidden, batch_size=n,
         activation=activation, m_norm_max=m_norm_max)
    return f, g


def host_swa_forward(q, k, v, num_heads, head_dim, window):
    q, k, v = map(_h, (q, k, v))
    s = q.shape[0]
    out = np.empty_like(q)
    aw = np.empty((num_heads, s, window), np.float32)
    call("nlh_swa_forward_dispatch", q=_hp(q), k=_hp(k), v=_hp(v), out=_hp(out), attn_weights=_hp(aw),
         seq_len=s, num_heads=num_heads, head_dim=head_dim, window_size=window)
    return {"out": out, "attn_weights": aw}


def host_swa_backward(q, k, v, attn_weights, d_out, num_heads, head_dim, window):
    q, k, v, d_out = map(_h, (q, k, v, d_out))
    s = q.shape[0]
    g = {n: np.zeros_like(q) for n in ("d_q", "d_k", "d_v")}
    call("nlh_swa_backward_dispatch", q=_hp(q), k=_hp(k), v=_hp(v),
         attn_weights=None if attn_weights is None else _hp(_h(attn_weights)), d_attn_out=_hp(d_out),
         d_q=_hp(g["d_q"]), d_k=_hp(g["d_k"]), d_v=_hp(g["d_v"]), seq_len=s, num_heads=num_heads,
         head_dim=head_dim, window_size=window)
    return g
