"""Single-block MAG model with one memory level (k = 1) on this library's kernels — the
reference's CPU-runnable configuration (core/src/mag.rs:74-392 mag_forward / mag_backward:
Delta rule or Titans LMM + MAG, one d_model x d_model memory, SWA branch gated by the memory
output). Host-side harness in the style of stacked_mag.py: the memory rule, SWA, the rule
wrapper (L2 norm, gates, head layout) and the cross-entropy run as opaque blocks of PyTorch's
tape through the C ABI; the dense projections are fp32 PyTorch matmuls.

Follows the CPU reference where its CPU and GPU paths differ: ONE memory of size d_model
(core/src/mag.rs:120-125), memory projections multiply by the bf16-rounded copy of
W_{k,v,q}_mem while the gradient goes to the fp32 master (core/src/bf16.rs:54-115), gate -> k/v
gradient included, M_0 = S_0 = 0 for every sequence. With fp32_swa (default) the attention runs
in fp32 like the reference's CPU path (core/src/swa.rs:33-235), so the whole configuration is
fp32; fp32_swa = False rounds q, k, v to bf16 and runs the tensor-core pair like the reference's
GPU dispatch (core/src/dispatch.rs:478-560).
"""
from __future__ import annotations

import torch

from . import dispatch as D
from .stacked_mag import _CrossEntropy, _LevelPrep, _SWA, _TitansMemory


class _DeltaMemory(torch.autograd.Function):
    """Delta rule over [N, S, d] (delta_forward_f32_cuda / delta_backward_f32_cuda), M_0 given."""

    @staticmethod
    def forward(ctx, k, v, q, alpha, theta, m0):
        ms, y = D.delta_forward_dd(k, v, q, alpha, theta, m0)
        ctx.save_for_backward(k, v, q, alpha, theta, ms)
        return y

    @staticmethod
    def backward(ctx, dy):
        k, v, q, alpha, theta, ms = ctx.saved_tensors
        g = D.delta_backward_dd(k, v, q, alpha, theta, ms, dy.contiguous())
        return g["d_k"], g["d_v"], g["d_q"], g["d_alpha"], g["d_theta"], None


def _bf16_weights(w):
    """Value: the bf16-rounded weights (as fp32); gradient: straight through to the master."""
    return w + (w.to(torch.bfloat16).float() - w).detach()


class MAGSingle:
    """params: dict of fp32 arrays keyed by the reference's MAGParams field names: w_embed [vocab, d],
    w_unembed [d, vocab], w_q, w_k, w_v, w_o, w_k_mem, w_v_mem, w_q_mem [d, d], w_alpha, w_theta
    (and w_eta for Titans) [2d], b_alpha, b_theta (b_eta) [1]."""

    def __init__(self, params, num_heads, window, rule="delta", device="cuda", fp32_swa=True):
        self.fp32_swa = fp32_swa
        self.p = {n: torch.as_tensor(a, dtype=torch.float32).to(device).clone().requires_grad_(True)
                  for n, a in params.items()}
        self.num_heads, self.window, self.rule = num_heads, window, rule

    def loss(self, input_ids, target_ids):
        """Mean cross-entropy over all positions of input_ids [B, S] (sequences are independent:
        every one starts from an empty memory)."""
        p = self.p
        B, S = input_ids.shape
        vocab, d = p["w_embed"].shape
        hd = d // self.num_heads
        emb = p["w_embed"][input_ids]                                       # [B, S, d]
        sdt = torch.float32 if self.fp32_swa else torch.bfloat16
        q, k, v = (torch.nn.functional.linear(emb, p[n]).to(sdt).contiguous()
                   for n in ("w_q", "w_k", "w_v"))
        attn = _SWA.apply(q, k, v, self.num_heads, hd, self.window).float()
        w_kvq = torch.cat([_bf16_weights(p[n]) for n in ("w_k_mem", "w_v_mem", "w_q_mem")], dim=0)
        kvq = torch.nn.functional.linear(emb, w_kvq)                        # [B, S, 3d] rows k | v | q
        zero_w, zero_b = torch.zeros_like(p["w_alpha"]), torch.zeros(1, device=emb.device)
        titans = self.rule == "titans"
        w_gates = torch.stack([p["w_alpha"], p["w_theta"], p["w_eta"] if titans else zero_w])
        km, vm, qm, alpha, theta, eta = _LevelPrep.apply(kvq, w_gates, p["b_alpha"], p["b_theta"],
                                                         p["b_eta"] if titans else zero_b, 1, 0)
        m0 = torch.zeros(B, d * d, device=emb.device)
        if titans:
            y, _ = _TitansMemory.apply(km, vm, qm, alpha, theta, eta, m0, 0, 0)
        else:
            y = _DeltaMemory.apply(km, vm, qm, alpha, theta, m0)
        gated = attn * torch.sigmoid(y.view(B, S, d))
        logits = torch.nn.functional.linear(gated, p["w_o"]) @ p["w_unembed"]
        return _CrossEntropy.apply(logits.view(B * S, vocab).contiguous(),
                                   target_ids.reshape(-1).to(torch.int32))

    def loss_and_grads(self, input_ids, target_ids):
        for w in self.p.values():
            w.grad = None
        loss = self.loss(input_ids, target_ids)
        loss.backward()
        return float(loss.detach()), {n: w.grad.detach().clone() for n, w in self.p.items() if w.grad is not None}
