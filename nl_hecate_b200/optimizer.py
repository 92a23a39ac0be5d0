"""Flat-arena AdamW for the outer parameters.

Host-side mirror of the per-tensor loop in
core/src/gpu_stacked_optimizer.rs:522-683 (``gpu_stacked_adamw_update``) and of
``FrequencyAwareAdamW::step`` (core/src/adamw.rs:195-395): all parameters, their
gradients and both moments live in four flat fp32 arenas with one layout, so
that the step is ONE global-norm reduction and ONE multi-tensor kernel (and,
data-parallel, ONE all-reduce over ``g``). Per-tensor state that the reference
keeps in separate launches travels in a descriptor table: the tensor's own
bias corrections (shared tensors use the global step, CMS level tensors their
level's fire count), whether it is active this step (pulse gating), and the
post-update clamp (``b_theta`` in [-10, 2]).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import ffi
from .dispatch import call

CHUNK = 8192  # elements per CTA work item


class FlatAdamW:
    def __init__(self, sizes, device="cuda", beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1,
                 clamp=None, no_decay=()):
        self.sizes = [int(s) for s in sizes]
        self.beta1, self.beta2, self.eps, self.weight_decay = beta1, beta2, eps, weight_decay
        self.clamp = dict(clamp or {})
        self.no_decay = set(no_decay)
        self.slices = []
        off = 0
        for n in self.sizes:
            self.slices.append((off, n))
            off += (n + 7) // 8 * 8          # 32-byte aligned in fp32, 16-byte aligned in a bf16 shadow of the arena
        self.arena_len = max(off, 4)
        dev = torch.device(device)
        z = lambda: torch.zeros(self.arena_len, dtype=torch.float32, device=dev)
        self.w, self.g, self.m, self.v = z(), z(), z(), z()
        ct, cs, cl = [], [], []
        for ti, (o, n) in enumerate(self.slices):
            for c0 in range(0, n, CHUNK):
                ct.append(ti); cs.append(o + c0); cl.append(min(CHUNK, n - c0))
        self.n_chunks = len(ct)
        self.chunk_tensor = torch.tensor(ct, dtype=torch.int32, device=dev)
        self.chunk_start = torch.tensor(cs, dtype=torch.int64, device=dev)
        self.chunk_len = torch.tensor(cl, dtype=torch.int32, device=dev)
        self._desc_host = (ffi.AdamWTensorDesc * len(self.sizes))()
        nbytes = C.sizeof(self._desc_host)
        self._desc_pinned = torch.empty(nbytes, dtype=torch.uint8)
        if dev.type == "cuda":
            self._desc_pinned = self._desc_pinned.pin_memory()
        self._desc_dev = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self._partial = torch.empty(148 * 8, dtype=torch.float32, device=dev)
        self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.scale = torch.ones(1, dtype=torch.float32, device=dev)
        # recorded after the stream-ordered upload of the pinned table in launch(); prepare()
        # waits on it before it rewrites the table, so a host that runs ahead of the GPU cannot
        # replace step t's descriptors before step t's copy has read them
        self._uploaded = torch.cuda.Event() if dev.type == "cuda" else None
        self._upload_pending = False

    def view(self, arena: torch.Tensor, i: int) -> torch.Tensor:
        o, n = self.slices[i]
        return arena[o:o + n]

    def prepare(self, steps, active=None, lr_scale=1.0):
        """Host part of a step: fill the per-tensor descriptor table (bias corrections from each
        tensor's own 1-based step count, activity, clamp, learning-rate scale) in pinned memory.
        The device reads it in launch(); a second prepare() first waits until the previous
        launch()'s upload of the table has completed."""
        if self._upload_pending:
            self._uploaded.synchronize()
            self._upload_pending = False
        nt = len(self.sizes)
        active = [True] * nt if active is None else active
        for i in range(nt):
            d = self._desc_host[i]
            t = max(int(steps[i]), 1)
            d.bc1_inv = 1.0 / (1.0 - self.beta1 ** t)
            d.bc2_inv = 1.0 / (1.0 - self.beta2 ** t)
            d.weight_decay = 0.0 if i in self.no_decay else self.weight_decay
            d.lr_scale = lr_scale
            lo, hi = self.clamp.get(i, (0.0, 0.0))
            d.clamp_lo, d.clamp_hi, d.has_clamp = lo, hi, int(i in self.clamp)
            d.active = int(bool(active[i]))
        C.memmove(self._desc_pinned.data_ptr(), C.addressof(self._desc_host),
                  C.sizeof(self._desc_host))

    def launch(self, lr, max_grad_norm=0.0):
        """Device part of a step (stream-ordered, capturable in a CUDA graph): descriptor upload,
        global-norm clip scale, multi-tensor AdamW. Returns the device scalar with the pre-clip
        gradient norm (valid only when max_grad_norm > 0)."""
        self._desc_dev.copy_(self._desc_pinned, non_blocking=True)
        if self._uploaded is not None and not torch.cuda.is_current_stream_capturing():
            self._uploaded.record()
            self._upload_pending = True
        scale_ptr = None
        if max_grad_norm > 0.0:
            call("nlh_arena_grad_norm_clip", g=self.g, n=self.arena_len,
                 max_grad_norm=max_grad_norm, partial=self._partial,
                 partial_capacity=self._partial.numel(), out_norm=self.norm, out_scale=self.scale)
            scale_ptr = self.scale
        call("nlh_adamw_multi_tensor", w=self.w, g=self.g, m=self.m, v=self.v,
             descs_dev=self._desc_dev, chunk_tensor_dev=self.chunk_tensor,
             chunk_start_dev=self.chunk_start, chunk_len_dev=self.chunk_len,
             n_chunks=self.n_chunks, grad_scale_ptr=scale_ptr, lr=lr, beta1=self.beta1,
             beta2=self.beta2, eps=self.eps)
        return self.norm

    def step(self, lr, steps, active=None, max_grad_norm=0.0):
        """One optimizer step. ``steps[i]`` is tensor i's own 1-based step count (bias
        correction), ``active[i]`` False skips it."""
        self.prepare(steps, active)
        return self.launch(lr, max_grad_norm)
