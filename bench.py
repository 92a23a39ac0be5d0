#!/usr/bin/env python
"""Benchmark of the NL_Hecate hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0). A "step" is one forward+backward pass of the
workload over one batch of seeded synthetic input:

  titans_chunkwise  Titans LMM frozen-M0 chunkwise kernel pair alone: batch 16 x 8 heads,
                    head_dim 64, seq 2048, chunk 64, fp32 (128 independent problems / GPU)
  titans_exact      same shapes, exact per-token rule (full-trajectory drop-in pair)
  swa               SWA forward+backward pair: bf16, batch 8 x 16 heads, head_dim 64,
                    seq 8192, causal window 512
  titans_level0     exact Titans pair at the stacked model's level-0 shape (512 problems of 512
                    tokens, M-only trajectory)
  titans_level1     frozen-M0 Titans pair at the stacked model's level-1 shape (512 problems of 64
                    pooled tokens, chunk 8, every state stored, streaming backward)
  adamw             flat-arena clip + AdamW step over 25.2 M fp32 parameters
--small shrinks the kernel-pair workloads to a profiler-friendly problem count.

`value` is device-timed (CUDA events on the launching stream, max over ranks) with
inputs resident in HBM; `e2e` goes through the host-slice API: pinned host buffers,
H2D of every input and D2H of every output inside the timed region. `--impl reference`
times the CPU restatement of the reference's Rust path (oracle/) on all host cores on
a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LOG2E = 1.4426950408889634


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                 "100", "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ─────────────────────────── workload definitions ───────────────────────────
class TitansPair:
    """Titans LMM kernel pair alone. chunk > 0: frozen-M0 chunkwise; chunk == 0: exact."""
    B, H, S, D = 16, 8, 2048, 64

    def __init__(self, chunk: int):
        self.chunk = chunk
        self.N = self.B * self.H
        self.name = "titans_chunkwise" if chunk else "titans_exact"
        self.tokens_per_step = self.B * self.S
        self.dtype = "f32"

    def describe(self):
        return {"workload": f"Titans LMM kernel pair ({'frozen-M0 chunkwise, chunk 64' if self.chunk else 'exact per-token, full trajectory'}): "
                            f"batch {self.B} x heads {self.H}, head_dim {self.D}, seq {self.S}, fp32",
                "problems_per_gpu": self.N, "tokens_per_step_per_gpu": self.tokens_per_step,
                "l2_policy": "inputs+outputs > L2 (>= 0.9 GB touched per step)"}

    def host_inputs(self, n=None, seed=1234):
        n = self.N if n is None else n
        g = np.random.Generator(np.random.Philox(seed))
        nrm = lambda x: (x / np.linalg.norm(x, axis=-1, keepdims=True)).astype(np.float32)
        sig = lambda x: (1.0 / (1.0 + np.exp(-x))).astype(np.float32)
        sh = (n, self.S, self.D)
        return dict(k=nrm(g.standard_normal(sh)), v=nrm(g.standard_normal(sh)),
                    q=nrm(g.standard_normal(sh)), alpha=sig(g.standard_normal(sh[:2])),
                    theta=sig(g.standard_normal(sh[:2])), eta=sig(g.standard_normal(sh[:2])),
                    dy=g.standard_normal(sh).astype(np.float32),
                    m0=np.zeros((n, self.D * self.D), np.float32),
                    s0=np.zeros((n, self.D * self.D), np.float32))

    def setup(self, torch, dispatch):
        self.torch, self.dd = torch, dispatch
        self.host = {k: torch.from_numpy(v).pin_memory() for k, v in self.host_inputs().items()}
        self.dev = {k: v.cuda() for k, v in self.host.items()}
        n, s, d = self.N, self.S, self.D
        f32 = lambda *sh: torch.empty(*sh, dtype=torch.float32, device="cuda")
        slots = (s // self.chunk + 1) if self.chunk else (s + 1)
        self.mstate, self.sstate, self.y = f32(n, slots, d * d), f32(n, slots, d * d), f32(n, s, d)
        self.out = {k: f32(n, s, d) for k in ("d_k", "d_v", "d_q")}
        self.out.update({k: f32(n, s) for k in ("d_alpha", "d_theta", "d_eta")})
        self.out.update({k: f32(d * d) for k in ("d_m0", "d_s0")})
        self.host_out = {k: torch.empty(v.shape, dtype=v.dtype).pin_memory()
                         for k, v in list(self.out.items()) + [("y", self.y)]}
        self.launches_per_step = 2
        self.h2d = sum(v.numel() * 4 for k, v in self.host.items())
        self.d2h = sum(v.numel() * 4 for v in self.host_out.values())

    def fwd(self, t):
        c = self.dd.call
        if self.chunk:
            c("titans_chunkwise_forward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"],
              alpha=t["alpha"], theta=t["theta"], eta=t["eta"], m_initial=t["m0"], s_initial=t["s0"],
              m_chunk_states=self.mstate, s_chunk_states=self.sstate, y=self.y, seq_len=self.S,
              d=self.D, batch_size=self.N, chunk_size=self.chunk, error_clip=0.0, m_norm_max=0.0)
        else:
            c("titans_forward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
              theta=t["theta"], eta=t["eta"], m_initial=t["m0"], s_initial=t["s0"],
              m_states=self.mstate, s_states=self.sstate, y=self.y, seq_len=self.S, d=self.D,
              batch_size=self.N, input_stride=self.S, m_stride=self.D * self.D, error_clip=0.0,
              m_norm_max=0.0)

    def bwd(self, t):
        c, o = self.dd.call, self.out
        o["d_m0"].zero_(); o["d_s0"].zero_()
        if self.chunk:
            c("titans_chunkwise_backward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"],
              alpha=t["alpha"], theta=t["theta"], eta=t["eta"], m_chunk_states=self.mstate,
              s_chunk_states=self.sstate, d_y=t["dy"], d_k_mem=o["d_k"], d_v_mem=o["d_v"],
              d_q_mem=o["d_q"], d_alpha=o["d_alpha"], d_theta=o["d_theta"], d_eta=o["d_eta"],
              d_m_initial=o["d_m0"], d_s_initial=o["d_s0"], seq_len=self.S, d=self.D,
              batch_size=self.N, chunk_size=self.chunk, error_clip=0.0, m_norm_max=0.0)
        else:
            c("titans_backward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
              theta=t["theta"], eta=t["eta"], m_states=self.mstate, s_states=self.sstate,
              d_y=t["dy"], d_k_mem=o["d_k"], d_v_mem=o["d_v"], d_q_mem=o["d_q"],
              d_alpha=o["d_alpha"], d_theta=o["d_theta"], d_eta=o["d_eta"], d_m_initial=o["d_m0"],
              d_s_initial=o["d_s0"], seq_len=self.S, d=self.D, batch_size=self.N, error_clip=0.0)

    def step(self):
        self.fwd(self.dev); self.bwd(self.dev)

    def step_e2e(self):
        t = {k: v.cuda(non_blocking=True) for k, v in self.host.items()}
        self.fwd(t); self.bwd(t)
        for k, v in self.out.items():
            self.host_out[k].copy_(v, non_blocking=True)
        self.host_out["y"].copy_(self.y, non_blocking=True)

    def dominant(self):
        """(name, callable, algorithmic bytes per launch, bound). Backward kernel."""
        n, s, d = self.N, self.S, self.D
        stream4 = 4 * n * s * d * 4            # k,v,q,d_y read
        out3 = 3 * n * s * d * 4               # d_k,d_v,d_q written
        gates = 6 * n * s * 4                  # 3 gates read + 3 gate grads written
        if self.chunk:
            states = 2 * n * (s // self.chunk + 1) * d * d * 4
        else:
            states = 2 * n * (s + 1) * d * d * 4
        return ("cmm::chunk_mm_bwd_kernel<TITANS> (frozen-M0 backward, chunk-parallel matrix form)" if self.chunk
                else "fast_bwd_kernel<64,TITANS,exact>",
                lambda: self.bwd(self.dev), stream4 + out3 + gates + states, "hbm")

    def cpu_sample(self, oracle, threads, budget_s=12.0):
        import ctypes as C
        d, s = self.D, self.S

        def run(nprob):
            p = self.host_inputs(nprob, seed=99)
            z = lambda *sh: np.zeros(sh, np.float32)      # zeros: pages are touched before the clock starts
            L = oracle.lib()
            ptr = oracle._p
            slots = (s // self.chunk + 1) if self.chunk else (s + 1)
            out = [z(nprob, slots, d * d), z(nprob, slots, d * d)] + [z(nprob, s, d) for _ in range(4)] + \
                  [z(nprob, s) for _ in range(3)] + [z(nprob, d * d), z(nprob, d * d)]
            t0 = time.perf_counter()
            if self.chunk:
                L.orc_chunkwise_fwd_bwd_batched_mt(
                    C.c_int(1), ptr(p["k"]), ptr(p["v"]), ptr(p["q"]), ptr(p["alpha"]), ptr(p["theta"]),
                    ptr(p["eta"]), ptr(p["m0"]), ptr(p["s0"]), ptr(p["dy"]), *[ptr(a) for a in out],
                    C.c_int(nprob), C.c_int(s), C.c_int(d), C.c_int(self.chunk), C.c_float(0.0),
                    C.c_float(0.0), C.c_int(threads))
            else:
                L.orc_titans_fwd_bwd_batched_mt(
                    ptr(p["k"]), ptr(p["v"]), ptr(p["q"]), ptr(p["alpha"]), ptr(p["theta"]),
                    ptr(p["eta"]), ptr(p["m0"]), ptr(p["s0"]), ptr(p["dy"]), *[ptr(a) for a in out],
                    C.c_int(nprob), C.c_int(s), C.c_int(d), C.c_float(0.0), C.c_float(0.0),
                    C.c_int(threads))
            return time.perf_counter() - t0
        t1 = run(threads)                              # one problem per thread
        reps = max(1, min(64 if s < 256 else 8, int(budget_s / max(t1, 1e-3)) - 1))
        nprob = threads * reps
        dt = run(nprob) if reps > 1 else t1
        head_tokens = nprob * s
        # tokens = sequence positions of the [B,S] batch = head-tokens / H
        return head_tokens / self.H / dt, (f"{nprob} of {self.N} (batch x head) problems, seq {s}, one problem at a time "
                                           f"per host thread: {dt:.1f} s (inputs and outputs allocated before the clock)")


class SwaPair:
    B, H, S, HD, W = 8, 16, 8192, 64, 512

    def __init__(self):
        self.name = "swa"
        self.tokens_per_step = self.B * self.S
        self.dtype = "bf16"

    def describe(self):
        return {"workload": f"SWA forward+backward pair: bf16, batch {self.B} x heads {self.H}, "
                            f"head_dim {self.HD}, seq {self.S}, causal window {self.W}",
                "tokens_per_step_per_gpu": self.tokens_per_step,
                "l2_policy": "inputs+outputs > L2 (1.9 GB touched per step)"}

    def host_inputs(self, b=None, seed=31):
        b = self.B if b is None else b
        g = np.random.Generator(np.random.Philox(seed))
        sh = (b, self.S, self.H * self.HD)
        mk = lambda: (g.standard_normal(sh) / 8.0).astype(np.float32)
        return dict(q=mk(), k=mk(), v=mk(), do=g.standard_normal(sh).astype(np.float32))

    def setup(self, torch, dispatch):
        self.torch, self.dd = torch, dispatch
        h = self.host_inputs()
        self.host = {k: (torch.from_numpy(v).bfloat16() if k != "do" else torch.from_numpy(v)).pin_memory()
                     for k, v in h.items()}
        self.dev = {k: v.cuda() for k, v in self.host.items()}
        sh = (self.B, self.S, self.H * self.HD)
        self.o = torch.empty(sh, dtype=torch.bfloat16, device="cuda")
        self.lse = torch.empty(self.B, self.H, self.S, dtype=torch.float32, device="cuda")
        self.g = {k: torch.empty(sh, dtype=torch.float32, device="cuda") for k in ("dq", "dk", "dv")}
        self.host_out = {k: torch.empty(sh, dtype=torch.float32).pin_memory() for k in self.g}
        self.host_out["out"] = torch.empty(sh, dtype=torch.bfloat16).pin_memory()
        self.launches_per_step = 4   # fwd, delta, dK/dV, dQ
        self.h2d = sum(v.numel() * v.element_size() for v in self.host.values())
        self.d2h = sum(v.numel() * v.element_size() for v in self.host_out.values())

    def fwd(self, t):
        self.dd.call("nlh_swa_forward", q=t["q"], k=t["k"], v=t["v"], out=self.o, lse=self.lse,
                     seq_len=self.S, num_heads=self.H, head_dim=self.HD, window_size=self.W,
                     batch_size=self.B, n_persistent=0)

    def bwd(self, t):
        self.dd.call("nlh_swa_backward", q=t["q"], k=t["k"], v=t["v"], out=self.o, lse=self.lse,
                     d_attn_out=t["do"], d_q=self.g["dq"], d_k=self.g["dk"], d_v=self.g["dv"],
                     seq_len=self.S, num_heads=self.H, head_dim=self.HD, window_size=self.W,
                     batch_size=self.B, n_persistent=0)

    def step(self):
        self.fwd(self.dev); self.bwd(self.dev)

    def step_e2e(self):
        t = {k: v.cuda(non_blocking=True) for k, v in self.host.items()}
        self.fwd(t); self.bwd(t)
        for k, v in self.g.items():
            self.host_out[k].copy_(v, non_blocking=True)
        self.host_out["out"].copy_(self.o, non_blocking=True)

    def dominant(self):
        pairs = (self.S * self.W - self.W * (self.W - 1) // 2) * self.B * self.H
        flops = pairs * (4 + 10) * self.HD      # fwd 4*hd + bwd 10*hd flop per visible (q,k) pair
        return ("swa fwd+bwd (4 launches)", lambda: self.step(), flops, "tensor")

    def cpu_sample(self, oracle, threads, budget_s=12.0):
        import ctypes as C
        # bounded sample: `threads` sequences (one per host thread) of seq 1024 with the same
        # window and head shape; attention work per token is the same once seq >= window
        s, nh, hd, w = 1024, self.H, self.HD, self.W
        g = np.random.Generator(np.random.Philox(5))
        sh = (threads, s, nh * hd)
        q, k, v = ((g.standard_normal(sh) / 8).astype(np.float32) for _ in range(3))
        do = g.standard_normal(sh).astype(np.float32)
        o = lambda *shape: np.zeros(shape, np.float32)
        ptr = oracle._p
        bufs = [o(*sh), o(threads, nh, s, w), o(*sh), o(*sh), o(*sh)]
        t0 = time.perf_counter()
        oracle.lib().orc_swa_fwd_bwd_batched_mt(
            ptr(q), ptr(k), ptr(v), ptr(do), *[ptr(a) for a in bufs], C.c_int(threads), C.c_int(s),
            C.c_int(nh), C.c_int(hd), C.c_int(w), C.c_int(0), C.c_int(threads))
        dt = time.perf_counter() - t0
        return threads * s / dt, f"{threads} sequences of seq {s} (window {w}, {nh} heads), {dt:.1f} s"


class AdamWStep:
    N_PARAMS = 25_200_000

    def __init__(self):
        self.name = "adamw"
        self.tokens_per_step = 64 * 512     # tokens of the cfg3 step this optimizer step serves
        self.dtype = "f32"

    def describe(self):
        return {"workload": f"flat-arena global-norm clip + AdamW step, {self.N_PARAMS} fp32 parameters",
                "tokens_per_step_per_gpu": self.tokens_per_step,
                "l2_policy": "4 arenas x 101 MB > L2"}

    def setup(self, torch, dispatch):
        from nl_hecate_b200.optimizer import FlatAdamW
        self.torch = torch
        sizes = [4_194_304, 4_194_304] + [262_144] * 16 + [789_507] * 16 + [1024] * 8
        sizes.append(self.N_PARAMS - sum(sizes))
        self.opt = FlatAdamW(sizes, device="cuda")
        g = torch.Generator(device="cuda").manual_seed(7)
        self.opt.w.normal_(0, 0.02, generator=g)
        self.opt.g.normal_(0, 0.01, generator=g)
        self.steps = [1] * len(sizes)
        self.host_g = torch.empty(self.opt.arena_len, dtype=torch.float32).pin_memory().normal_(0, 0.01)
        self.host_norm = torch.empty(1, dtype=torch.float32).pin_memory()
        self.launches_per_step = 3
        self.h2d = self.opt.arena_len * 4
        self.d2h = 4
        self.t = 0

    def step(self):
        self.t += 1
        self.opt.step(lr=3e-4, steps=[self.t] * len(self.steps), max_grad_norm=1.0)

    def step_e2e(self):
        self.opt.g.copy_(self.host_g, non_blocking=True)
        self.step()
        self.host_norm.copy_(self.opt.norm, non_blocking=True)

    def dominant(self):
        return ("adamw_multi_kernel + arena_sumsq_kernel", lambda: self.step(),
                self.opt.arena_len * 32, "hbm")   # 4 B norm pass + 16 B read + 12 B written

    def cpu_sample(self, oracle, threads, budget_s=12.0):
        import ctypes as C
        n = self.N_PARAMS
        w, g, m, v = (np.full(n, x, np.float32) for x in (0.01, 0.001, 0.0, 0.0))
        ptr = oracle._p
        t0 = time.perf_counter()
        reps = 3
        for _ in range(reps):
            oracle.lib().orc_adamw_step_mt(ptr(w), ptr(g), ptr(m), ptr(v), C.c_int64(n),
                                           C.c_float(3e-4), C.c_float(0.9), C.c_float(0.999),
                                           C.c_float(1e-8), C.c_float(10.0), C.c_float(1000.0),
                                           C.c_float(0.1), C.c_int(threads))
        dt = (time.perf_counter() - t0) / reps
        return self.tokens_per_step / dt, f"{reps} full steps over {n} parameters, {dt * 1e3:.0f} ms each"


class StackedModelStep:
    """Full model step (configuration the headline metric is quoted on): Titans LMM + MAG + SWA
    (window 512), CMS k=4 with periods [1,8,64,512], d_model 512, 8 heads, 4 blocks, vocab 8192,
    seq 512, GLOBAL batch 64 split over the ranks; bf16 activations, fp32 memory state;
    forward + backward + gradient all-reduce + clip + AdamW."""
    GLOBAL_BATCH, S, VOCAB = 64, 512, 8192

    def __init__(self, world, local_batch=0):
        self.name = "stacked_mag"
        self.world = world
        assert self.GLOBAL_BATCH % world == 0
        # local_batch > 0 (--local-batch): run the per-rank shard of a larger job on this GPU alone,
        # e.g. 8 sequences = one rank of the 8-GPU run, to profile that shape without 8 GPUs
        self.local_batch = local_batch if local_batch > 0 else self.GLOBAL_BATCH // world
        self.tokens_per_step = self.local_batch * self.S
        self.dtype = "bf16"

    def describe(self):
        return {"workload": "full model step: Titans LMM + MAG + SWA(window 512), CMS k=4 periods "
                            "[1,8,64,512], d_model 512, 8 heads, 4 blocks, vocab 8192, seq 512, "
                            f"global batch {self.GLOBAL_BATCH}; fwd+bwd+all-reduce+clip+AdamW; bf16 "
                            "activations, fp32 memory state; static projections",
                "global_batch": self.GLOBAL_BATCH, "seq_len": self.S,
                "tokens_per_step_per_gpu": self.tokens_per_step,
                "l2_policy": "per-step working set (tens of GB of memory-state trajectory) >> L2"}

    def zipf_tokens(self, n_seq, seed=2024):
        g = np.random.Generator(np.random.Philox(seed))
        ranks = np.arange(1, self.VOCAB + 1, dtype=np.float64)
        cdf = np.cumsum(ranks ** -1.1)
        cdf /= cdf[-1]
        ids = np.searchsorted(cdf, g.random((n_seq, self.S + 1)), side="left").astype(np.int64)
        return np.minimum(ids, self.VOCAB - 1)

    def setup(self, torch, dispatch):
        from nl_hecate_b200.stacked_mag import StackedMAG, StackedMAGConfig
        self.torch, self.dd = torch, dispatch
        rank = int(os.environ.get("RANK", "0"))
        self.cfg = StackedMAGConfig(level_streams=os.environ.get("NLH_BENCH_LEVEL_STREAMS", "1") == "1",
                                    overlap_grad_sync=os.environ.get("NLH_BENCH_OVERLAP", "1") == "1",
                                    exact_checkpoint=int(os.environ.get("NLH_BENCH_EXACT_CKPT", "0")))
        self.model = StackedMAG(self.cfg, self.local_batch, device="cuda", seed=42)
        ids = self.zipf_tokens(self.GLOBAL_BATCH)[rank * self.local_batch:(rank + 1) * self.local_batch]
        self.host_tok = torch.from_numpy(np.ascontiguousarray(ids[:, :-1])).pin_memory()
        self.host_tgt = torch.from_numpy(np.ascontiguousarray(ids[:, 1:])).pin_memory()
        self.tok, self.tgt = self.host_tok.cuda(), self.host_tgt.cuda()
        self.host_loss = torch.empty(1, dtype=torch.float32).pin_memory()
        # this library's launches per step (the profiler's launch list shows the same kernels).
        # Per block: SWA fwd (1) + bwd (3); MAG combine fwd + bwd + level-weight finisher (3); two
        # LayerNorms fwd + bwd (4; the second backward also upsamples the pooled levels' gradients);
        # one mean pool per pooled level (p); pooled-level output gradients (p); per level: prep
        # fwd (1) + bwd (3: d_kvq, gate weights, finisher), memory fwd + bwd (2). Once: final
        # LayerNorm (2), cross-entropy (2), embedding (2), gradient norm (2), AdamW (1).
        p = sum(1 for c in self.cfg.chunk_sizes[:self.cfg.k] if min(c, self.S) > 1)
        self.launches_per_step = self.cfg.n_blocks * (4 + 3 + 4 + p + p + 6 * self.cfg.k) + 9
        self.h2d = self.host_tok.numel() * 8 * 2
        self.d2h = 4
        self.pg = None
        self.use_graph = os.environ.get("NLH_BENCH_NO_GRAPH", "0") != "1"

    def step(self):
        if self.use_graph:
            return self.model.step_graphed(self.tok, self.tgt, self.pg, self.world)
        return self.model.step(self.tok, self.tgt, self.pg, self.world)

    def step_e2e(self):
        if self.use_graph:   # pinned host ids -> static device buffers -> graph replay -> loss to host
            loss = self.model.step_graphed(self.host_tok, self.host_tgt, self.pg, self.world)
        else:
            tok = self.host_tok.cuda(non_blocking=True)
            tgt = self.host_tgt.cuda(non_blocking=True)
            loss = self.model.step(tok, tgt, self.pg, self.world)
        self.host_loss.copy_(loss.reshape(1), non_blocking=True)

    def dominant(self):
        """Exact Titans backward at the level-0 shapes of one block (the kernel with the largest
        share of the step): N = local_batch x 8 heads problems, seq 512, head_dim 64."""
        torch = self.torch
        n, s, d = self.local_batch * self.cfg.num_heads, self.S, self.cfg.head_dim
        g = torch.Generator(device="cuda").manual_seed(5)
        r = lambda *sh: torch.randn(*sh, generator=g, device="cuda")
        k, v, q, dy = (torch.nn.functional.normalize(r(n, s, d), dim=-1) for _ in range(4))
        al, th, et = (torch.sigmoid(r(n, s)) for _ in range(3))
        m0 = torch.zeros(n, d * d, device="cuda")
        # as the model runs it: M trajectory only (s_states = NULL), S derived in the kernel
        ms, _, _ = self.dd.titans_forward_dd(k, v, q, al, th, et, m0, m0, store_s=False)
        bytes_ = (4 + 3) * n * s * d * 4 + 6 * n * s * 4 + n * (s + 1) * d * d * 4
        self._dom = (k, v, q, al, th, et, ms, dy)
        # DRAM bytes of one launch from the profiler capture of this kernel on a smaller case
        # (296 problems x 512 tokens: 2645.1 MB read + 113.5 MB written), scaled by problem-tokens
        # (the kernel reads each stored state once and streams the rest: traffic is proportional to them)
        self.dominant_traffic = (2_645_135_872 + 113_477_632) / (296 * 512) * n * s
        self.dominant_traffic_source = ("literal: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of "
                                        "this kernel at 296 problems x 512 tokens (bench.py --workload titans_level0 "
                                        "--small; profiles/titans_exact_level0_kernels.md), scaled by problem-tokens; "
                                        "not re-measured by this run")
        return ("titans_exact_bwd_kernel<64> (exact Titans backward, M-only trajectory) at level-0 shapes",
                lambda: self.dd.titans_backward_dd(k, v, q, al, th, et, ms, None, dy), bytes_, "hbm")

    def cpu_sample(self, oracle, threads, budget_s=12.0):
        """The SAME step on the host: the stacked-model oracle (oracle/stacked.py — embedding,
        LayerNorms, projections, SWA, four CMS levels of per-head Titans LMM, MAG gating,
        unembedding, cross-entropy, forward and backward) with the model's seeded initialisation on
        the first min(64, threads) sequences of the same Zipf token ids, one sequence per host
        thread and single-threaded inside a sequence (as the reference's Rust path runs), followed
        by gradient averaging, global-norm clip and one AdamW step over all parameters. Parameters,
        token ids and output buffers are prepared before the clock starts."""
        import ctypes as C
        from concurrent.futures import ThreadPoolExecutor
        from oracle import stacked as ST
        try:
            from threadpoolctl import threadpool_limits
        except ImportError:                                  # pragma: no cover
            threadpool_limits = None
        nseq = max(1, min(self.GLOBAL_BATCH, threads))
        cfg = ST.Cfg(d_model=512, num_heads=8, n_blocks=4, k=4, chunk_sizes=(1, 8, 64, 512), seq_len=self.S,
                     window=512, vocab=self.VOCAB, exact_levels=(0,), mode="resident")
        if getattr(self, "_cpu_params", None) is None:
            self._cpu_params = ST.init_params(cfg, seed=42)
            self._cpu_params["w_embed"] = np.ascontiguousarray(self._cpu_params["w_unembed"].T)   # tied
        p = self._cpu_params
        ids = self.zipf_tokens(self.GLOBAL_BATCH)[:nseq]
        if getattr(self, "_cpu_state", None) is None or len(self._cpu_state[0]) != nseq:
            # carried memories and trajectory buffers of the sampled sequence streams persist
            # from one timed step to the next, like the GPU arm's
            self._cpu_state = ([ST.new_context(cfg) for _ in range(nseq)], [dict() for _ in range(nseq)])
        ctxs, pools = self._cpu_state
        names = sorted(p)
        npar = sum(p[n].size for n in names)
        w_ = np.concatenate([p[n].ravel() for n in names]).astype(np.float32)
        g_, m_, v_ = (np.zeros(npar, np.float32) for _ in range(3))
        L, ptr = oracle.lib(), oracle._p

        def one(i):
            return ST.forward_backward(p, ids[i, :-1], ids[i, 1:], ctxs[i], cfg, pool=pools[i])

        import contextlib
        with (threadpool_limits(limits=1) if threadpool_limits else contextlib.nullcontext()):
            t0 = time.perf_counter()
            with ThreadPoolExecutor(max_workers=nseq) as ex:
                res = list(ex.map(one, range(nseq)))
            o = 0
            for n in names:                                  # average the per-sequence gradients
                acc = res[0][1][n].astype(np.float32).ravel().copy()
                for r in res[1:]:
                    acc += r[1][n].ravel()
                g_[o:o + acc.size] = acc / nseq
                o += acc.size
            scale = C.c_float(1.0)
            L.orc_grad_norm_clip(ptr(g_), C.c_int64(npar), C.c_float(1.0), C.byref(scale))
            L.orc_adamw_step_mt(ptr(w_), ptr(g_), ptr(m_), ptr(v_), C.c_int64(npar), C.c_float(3e-4),
                                C.c_float(0.9), C.c_float(0.999), C.c_float(1e-8), C.c_float(10.0),
                                C.c_float(1000.0), C.c_float(0.1), C.c_int(threads))
            dt = time.perf_counter() - t0
        loss = float(np.mean([r[0] for r in res]))
        return nseq * self.S / dt, (f"one whole step (embedding to AdamW, forward + backward, same seeded init and "
                                    f"token ids as the GPU arm) on {nseq} of {self.GLOBAL_BATCH} sequences, one per "
                                    f"host thread: {dt:.1f} s, {self.S / dt:.0f} tokens/s per thread, loss {loss:.4f}; "
                                    f"the {self.GLOBAL_BATCH}-sequence step time is extrapolated from it")


class TitansLevel0(TitansPair):
    """Exact Titans pair as level 0 of the stacked model runs it: 512 problems (64 sequences x 8
    heads) of 512 tokens, M-only trajectory (s_states = NULL), gates as the model's biases give."""
    B, H, S, D = 64, 8, 512, 64

    def __init__(self):
        super().__init__(0)
        self.name = "titans_level0"

    def describe(self):
        d = super().describe()
        d["workload"] = (f"Titans LMM exact pair at the stacked model's level-0 shape: batch {self.B} x heads "
                         f"{self.H}, head_dim {self.D}, seq {self.S}, fp32, M-only trajectory")
        return d

    def host_inputs(self, n=None, seed=1234):
        h = super().host_inputs(n, seed)
        g = np.random.Generator(np.random.Philox(seed + 7))
        sig = lambda x: (1.0 / (1.0 + np.exp(-x))).astype(np.float32)
        sh = h["alpha"].shape
        h["alpha"] = sig(g.standard_normal(sh) + 3.0)
        h["theta"] = np.log1p(np.exp(g.standard_normal(sh) - 4.6)).astype(np.float32)
        h["eta"] = sig(g.standard_normal(sh) + 1.5)
        return h

    def setup(self, torch, dispatch):
        super().setup(torch, dispatch)
        self.sstate = None                      # s_states = NULL: M-only trajectory

    def dominant(self):
        n, s, d = self.N, self.S, self.D
        streams = 7 * n * s * d * 4 + 6 * n * s * 4
        return ("titans_exact_bwd_kernel<64> (exact Titans backward, M-only trajectory)",
                lambda: self.bwd(self.dev), streams + n * (s + 1) * d * d * 4, "hbm")


class TitansLevel1(TitansLevel0):
    """Frozen-M0 Titans pair as level 1 of the stacked model runs it: 512 problems of 64 pooled
    tokens, chunk 8, every state stored and the backward streaming them (nlh_rule_forward /
    nlh_rule_backward with interval = 1)."""
    B, H, S, D = 64, 8, 64, 64
    CHUNK = 8

    def __init__(self):
        super().__init__()
        self.name = "titans_level1"

    def describe(self):
        d = super().describe()
        d["workload"] = (f"Titans LMM frozen-M0 pair (chunk {self.CHUNK}, full trajectory) at the stacked model's "
                         f"level-1 shape: batch {self.B} x heads {self.H}, head_dim {self.D}, seq {self.S}, fp32")
        d["l2_policy"] = "L2 flushed by the harness between steps is not needed: 0.55 GB of trajectory per step > L2"
        return d

    def fwd(self, t):
        self.dd.call("nlh_rule_forward", rule=1, k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
                     theta=t["theta"], eta=t["eta"], m_initial=t["m0"], s_initial=t["s0"], m_ckpt=self.mstate,
                     s_ckpt=None, y=self.y, seq_len=self.S, d=self.D, batch_size=self.N, interval=1,
                     chunk_size=self.CHUNK, error_clip=0.0, m_norm_max=0.0)

    def bwd(self, t):
        o = self.out
        self.dd.call("nlh_rule_backward", rule=1, k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
                     theta=t["theta"], eta=t["eta"], m_ckpt=self.mstate, s_ckpt=None, d_y=t["dy"],
                     d_k_mem=o["d_k"], d_v_mem=o["d_v"], d_q_mem=o["d_q"], d_alpha=o["d_alpha"],
                     d_theta=o["d_theta"], d_eta=o["d_eta"], d_m_initial=None, d_s_initial=None,
                     seq_len=self.S, d=self.D, batch_size=self.N, interval=1, chunk_size=self.CHUNK,
                     error_clip=0.0, m_norm_max=0.0)

    def dominant(self):
        n, s, d = self.N, self.S, self.D
        streams = 7 * n * s * d * 4 + 6 * n * s * 4
        return ("titans_exact_bwd_kernel<64,1,FROZEN> (frozen-M0 backward on the full M trajectory)",
                lambda: self.bwd(self.dev), streams + n * (s + 1) * d * d * 4, "hbm")

    def cpu_sample(self, oracle, threads, budget_s=12.0):
        self.chunk = self.CHUNK                      # the CPU arm runs the oracle's chunkwise rule
        try:
            return super().cpu_sample(oracle, threads, budget_s)
        finally:
            self.chunk = 0


class TitansMlpPair(TitansPair):
    """Titans LMM with a two-layer MLP memory (deep neural memory), kernel pair alone: the packed
    state W1[256,64] b1 W2[64,256] b2 per head, GELU, both trajectories stored as the ABI asks."""
    B, H, S, D, DH = 16, 8, 512, 64, 256

    def __init__(self):
        super().__init__(0)
        self.name = "titans_mlp"
        self.SS = self.DH * self.D * 2 + self.DH + self.D

    def describe(self):
        return {"workload": f"Titans LMM MLP-memory kernel pair (2 layers, d_hidden {self.DH}, GELU, full M and S "
                            f"trajectories): batch {self.B} x heads {self.H}, head_dim {self.D}, seq {self.S}, fp32",
                "problems_per_gpu": self.N, "tokens_per_step_per_gpu": self.tokens_per_step,
                "l2_policy": "trajectories written and read per step (2 x 132 KB per head-token) >> L2"}

    def host_inputs(self, n=None, seed=1234):
        n = self.N if n is None else n
        g = np.random.Generator(np.random.Philox(seed))
        nrm = lambda x: (x / np.linalg.norm(x, axis=-1, keepdims=True)).astype(np.float32)
        sig = lambda x: (1.0 / (1.0 + np.exp(-x))).astype(np.float32)
        sh = (n, self.S, self.D)
        return dict(k=nrm(g.standard_normal(sh)), v=(0.5 * g.standard_normal(sh)).astype(np.float32),
                    q=nrm(g.standard_normal(sh)), alpha=sig(g.standard_normal(sh[:2]) - 3.0),
                    theta=np.log1p(np.exp(g.standard_normal(sh[:2]) - 3.0)).astype(np.float32),
                    eta=sig(g.standard_normal(sh[:2]) + 1.5), dy=g.standard_normal(sh).astype(np.float32),
                    m0=(0.1 * g.standard_normal((n, self.SS))).astype(np.float32),
                    s0=np.zeros((n, self.SS), np.float32))

    def setup(self, torch, dispatch):
        self.torch, self.dd = torch, dispatch
        self.host = {k: torch.from_numpy(v).pin_memory() for k, v in self.host_inputs().items()}
        self.dev = {k: v.cuda() for k, v in self.host.items()}
        n, s, d = self.N, self.S, self.D
        f32 = lambda *sh: torch.empty(*sh, dtype=torch.float32, device="cuda")
        self.mstate, self.sstate, self.y = f32(n, s + 1, self.SS), f32(n, s + 1, self.SS), f32(n, s, d)
        self.out = {k: f32(n, s, d) for k in ("d_k", "d_v", "d_q")}
        self.out.update({k: f32(n, s) for k in ("d_alpha", "d_theta", "d_eta")})
        self.out.update({k: f32(self.SS) for k in ("d_m0", "d_s0")})
        self.host_out = {k: torch.empty(v.shape, dtype=v.dtype).pin_memory()
                         for k, v in list(self.out.items()) + [("y", self.y)]}
        self.launches_per_step = 2
        self.h2d = sum(v.numel() * 4 for k, v in self.host.items())
        self.d2h = sum(v.numel() * 4 for v in self.host_out.values())

    def fwd(self, t):
        self.dd.call("titans_mlp_forward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
                     theta=t["theta"], eta=t["eta"], m_initial=t["m0"], s_initial=t["s0"], m_states=self.mstate,
                     s_states=self.sstate, y=self.y, seq_len=self.S, d=self.D, d_hidden=self.DH, batch_size=self.N,
                     input_stride=self.S * self.D, m_stride=(self.S + 1) * self.SS, activation=0, m_norm_max=0.0)

    def bwd(self, t):
        o = self.out
        o["d_m0"].zero_(); o["d_s0"].zero_()
        self.dd.call("titans_mlp_backward_f32_cuda", k_mem=t["k"], v_mem=t["v"], q_mem=t["q"], alpha=t["alpha"],
                     theta=t["theta"], eta=t["eta"], m_states=self.mstate, s_states=self.sstate, d_y=t["dy"],
                     d_k_mem=o["d_k"], d_v_mem=o["d_v"], d_q_mem=o["d_q"], d_alpha=o["d_alpha"],
                     d_theta=o["d_theta"], d_eta=o["d_eta"], d_m_initial=o["d_m0"], d_s_initial=o["d_s0"],
                     seq_len=self.S, d=self.D, d_hidden=self.DH, batch_size=self.N, input_stride=self.S * self.D,
                     m_stride=(self.S + 1) * self.SS, activation=0, m_norm_max=0.0)

    def dominant(self):
        """Backward: reads k, v, q, d_y, gates and every stored M and S state once; writes d_k, d_v,
        d_q and the gate gradients."""
        n, s, d = self.N, self.S, self.D
        streams = 7 * n * s * d * 4 + 6 * n * s * 4
        # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel at 8 problems x 512
        # tokens (profiles/titans_mlp_memory_kernels.md); every stored state is read once: proportional to problems
        self.dominant_traffic = (1_091_155_968 + 3_302_144) / 8 * n
        self.dominant_traffic_source = ("literal: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                        "kernel at 8 problems x 512 tokens (bench.py --workload titans_mlp --small; "
                                        "profiles/titans_mlp_memory_kernels.md), scaled by problems; not re-measured by this run")
        return ("mlpm::s64::mlp_bwd64_kernel<GELU> (MLP-memory backward, M and S trajectories)",
                lambda: self.bwd(self.dev), streams + 2 * n * (s + 1) * self.SS * 4, "hbm")

    def cpu_sample(self, oracle, threads, budget_s=12.0):
        """The numpy restatement of the Rust path (oracle/mlp_memory.py), one problem per host
        process, shortened sequences of the same head size."""
        from concurrent.futures import ProcessPoolExecutor
        from oracle import mlp_memory
        s = 64
        jobs = [(1000 + i, s, self.D, self.DH, 0) for i in range(threads)]
        with ProcessPoolExecutor(max_workers=threads) as ex:
            list(ex.map(mlp_memory.timed_fwd_bwd, jobs))               # start the workers, import numpy
            t0 = time.perf_counter()
            list(ex.map(mlp_memory.timed_fwd_bwd, jobs))
            t1 = time.perf_counter() - t0
            reps = max(1, min(512, int(budget_s / max(t1, 1e-3))))
            jobs = [(2000 + i, s, self.D, self.DH, 0) for i in range(threads * reps)]
            t0 = time.perf_counter()
            done = sum(ex.map(mlp_memory.timed_fwd_bwd, jobs, chunksize=reps))
            dt = time.perf_counter() - t0
        return done / self.H / dt, (f"{threads * reps} (batch x head) problems of {s} tokens (of {self.N} x {self.S}), "
                                    f"{reps} per host process, numpy statement of the reference's Rust loop: {dt:.1f} s")


def make_workload(name, world=1, small=False, local_batch=0):
    """small: reduced problem counts of the same kernels, sized for profiler captures (inputs still
    larger than L2, a few hundred MB on the device)."""
    if small:
        TitansPair.B, SwaPair.B, TitansLevel0.B, TitansLevel1.B, TitansMlpPair.B = 4, 1, 37, 64, 1
    if name == "titans_chunkwise":
        return TitansPair(64)
    if name == "titans_exact":
        return TitansPair(0)
    if name == "titans_level0":
        return TitansLevel0()
    if name == "titans_level1":
        return TitansLevel1()
    if name == "titans_mlp":
        return TitansMlpPair()
    if name == "swa":
        return SwaPair()
    if name == "adamw":
        return AdamWStep()
    if name == "stacked_mag":
        return StackedModelStep(world, local_batch)
    raise SystemExit(f"unknown workload {name}")


DEFAULT_WORKLOAD = "stacked_mag"
METRIC = "fwd+bwd tokens/sec"
UNIT = "tokens/s"


def parallelism_label(workload, world):
    if workload == "stacked_mag":
        return f"dp{world} (batch shard, fp32 gradient all-reduce in per-block buckets under the backward)"
    return f"dp{world} (independent problems per rank, no collective)"


def run_reference(args):
    """CPU arm: the restated Rust reference path on all host threads, bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.build()
    wl = make_workload(args.workload, max(1, args.gpus))
    threads = oracle.hardware_threads()
    vals, secs = [], []
    sample = ""
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        v, sample = wl.cpu_sample(oracle, threads, budget_s=max(2.0, 20.0 / max(1, args.steps)))
        if i >= args.warmup:
            vals.append(v)
            secs.append(time.perf_counter() - t0)
    value = float(np.mean(vals))
    cfg = wl.describe()
    cfg["parallelism"] = parallelism_label(args.workload, max(1, args.gpus))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        # a step of this arm is one bounded sample of the workload: ms_per_step is its measured wall
        # time; the time a whole step of the configuration would take on these cores follows from
        # the throughput (sequences / problems are independent)
        "ms_per_step": 1e3 * float(np.mean(secs)),
        "full_step_ms_extrapolated": 1e3 * wl.tokens_per_step * max(1, args.gpus) / value,
        "higher_is_better": True,
        "scaling": "strong" if args.workload == "stacked_mag" else "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true",
                    help="kernel-pair workloads at a reduced problem count (profiler captures)")
    ap.add_argument("--local-batch", type=int, default=0,
                    help="stacked_mag only: sequences on this GPU instead of global batch / ranks "
                         "(profiles the per-rank shape of a multi-GPU run on one GPU)")
    ap.add_argument("--timed-only", action="store_true",
                    help="run only warm-up and the timed steps (for profiler launch lists)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from nl_hecate_b200 import dispatch, ffi
    ffi.lib()   # raises if the CUDA library is not built
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the CPU arm is --impl reference)")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        # The collective runs under the backward. Its kernels must fit on the SMs the level-0
        # kernels leave idle (128 of 148 busy at 4 and 8 ranks), or they slow the step's critical
        # path: 12 CTAs measured best at 2 and 4 ranks (4 ranks: 7.48 ms per step against 8.15 ms
        # with the library default and 7.47 ms with no overlap at all).
        os.environ.setdefault("NCCL_MAX_CTAS", "12")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    warmup = max(args.warmup, 3)

    wl = make_workload(args.workload, world, args.small, args.local_batch)
    wl.setup(torch, dispatch)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, k):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(k):
            fn()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(warmup):
        wl.step()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = timed(wl.step, args.steps)
    clocks = sampler.stop() if sampler else None
    tokens = wl.tokens_per_step * world * args.steps
    value = tokens / (ms * 1e-3)

    if args.timed_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
                              "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps,
                              "timed_only": True, "config": wl.describe()}))
        finish(world, barrier, wl)
        return

    # end to end through the host-slice API
    for _ in range(2):
        wl.step_e2e()
    ms_e2e = timed(wl.step_e2e, max(1, min(args.steps, 5)))
    e2e_value = wl.tokens_per_step * world * max(1, min(args.steps, 5)) / (ms_e2e * 1e-3)

    # roofline of the dominant kernel, timed alone with CUDA events on the launching stream
    peaks = measured_peaks()
    name, fn, work, bound = wl.dominant()
    for _ in range(3):
        fn()
    reps = max(3, min(args.steps, 10))
    ms_dom = timed(fn, reps) / reps
    if bound == "hbm":
        achieved = work / (ms_dom * 1e-3) / 1e9
        peak, runit = peaks["hbm_gbs"], "GB/s"
    else:
        achieved = work / (ms_dom * 1e-3) / 1e12
        peak, runit = peaks["bf16_tflops"], "TFLOP/s"
    roofline = {"kernel": name, "bound": bound, "achieved": achieved, "peak": peak, "unit": runit,
                "frac": achieved / peak, "traffic": getattr(wl, "dominant_traffic", None),
                "traffic_source": getattr(wl, "dominant_traffic_source", None),
                "ms_per_launch": ms_dom,
                "algorithmic_work_per_launch": work, "peak_source": peaks["source"]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        oracle.build()
        th = oracle.hardware_threads()
        v, sample = wl.cpu_sample(oracle, th)
        cpu = {"value": v, "unit": UNIT, "cores": th, "kind": "port", "sample": sample}

    if rank == 0:
        cfg = wl.describe()
        model_step = args.workload == "stacked_mag"
        cfg["parallelism"] = parallelism_label(args.workload, world)
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if model_step else "weak", "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic", "config": cfg, "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": wl.h2d,
                    "d2h_bytes_per_step": wl.d2h},
            "gpu_launches": wl.launches_per_step * args.steps,
            "roofline": roofline, "cpu_baseline": cpu,
        }))
    finish(world, barrier, wl)


def finish(world, barrier, wl):
    """End of a multi-rank run, in the order the resources depend on each other: every rank has
    printed / finished its work (barrier), the captured step graph — which holds the
    communicator's captured all-reduce — is dropped, the device is idle, and only then the
    process group is destroyed. A daemon timer ends the process if the teardown itself were to
    block for more than 30 s (the result line is already out)."""
    sys.stdout.flush()
    sys.stderr.flush()
    if world <= 1:
        return
    import torch
    import torch.distributed as dist
    watchdog = threading.Timer(30.0, lambda: os._exit(0))
    watchdog.daemon = True
    watchdog.start()
    barrier()
    model = getattr(wl, "model", None)
    if model is not None and getattr(model, "_graph", None) is not None:
        model._graph = None          # releases the captured collective before the communicator goes
    import gc
    gc.collect()
    torch.cuda.synchronize()
    dist.destroy_process_group()
    watchdog.cancel()


if __name__ == "__main__":
    main()
