"""Small stand-alone launches of single hot-path kernels, sized for profiler captures.

    python -m nl_hecate_b200.profile_cases titans_level0 [N] [S] [reps]
    python -m nl_hecate_b200.profile_cases swa_forward [B] [S] [H] [W] [tcgen05: 0|1]

Each case allocates well under a few GB, runs the kernels a few times through the C ABI and
prints CUDA-event times; run it once plainly, then under the profiler with a kernel filter.
"""
from __future__ import annotations

import sys

import torch
import torch.nn.functional as F

from . import dispatch as D


def titans_level0(n=296, s=128, reps=1):
    """Exact Titans pair as level 0 of the stacked model runs it: head_dim 64, M-only trajectory
    (s_states = NULL), gates from the model's initial biases."""
    d = 64
    g = torch.Generator(device="cuda").manual_seed(1)
    r = lambda *sh: torch.randn(*sh, device="cuda", generator=g)
    k, q, v = F.normalize(r(n, s, d), dim=-1), F.normalize(r(n, s, d), dim=-1), r(n, s, d) * 0.5
    alpha = torch.sigmoid(r(n, s) + 3).contiguous()
    theta = F.softplus(r(n, s) - 4.6).contiguous()
    eta = torch.sigmoid(r(n, s) + 1.5).contiguous()
    m0, s0, dy = torch.zeros(n, d * d, device="cuda"), torch.zeros(n, d * d, device="cuda"), r(n, s, d)
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    for _ in range(reps):
        e0.record()
        ms, _, _ = D.titans_forward_dd(k, v, q, alpha, theta, eta, m0, s0, store_s=False)
        e1.record()
        D.titans_backward_dd(k, v, q, alpha, theta, eta, ms, None, dy)
        e2.record()
        torch.cuda.synchronize()
        print(f"titans_level0 N={n} S={s}: forward {e0.elapsed_time(e1):.3f} ms, "
              f"backward (+ output zero fill) {e1.elapsed_time(e2):.3f} ms")


def swa_forward(b=8, s=8192, h=16, w=512, tc=1):
    hd = 64
    D.call("nlh_set_option", option=1, value=tc)
    q, k, v = ((torch.randn(b, s, h * hd, device="cuda") / 8).bfloat16() for _ in range(3))
    for _ in range(3):
        D.swa_forward_lse(q, k, v, h, hd, w)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        D.swa_forward_lse(q, k, v, h, hd, w)
    e1.record()
    torch.cuda.synchronize()
    pairs = (s * w - w * (w - 1) // 2 if s >= w else s * (s + 1) // 2) * b * h
    ms = e0.elapsed_time(e1) / 10
    print(f"swa_forward B={b} S={s} H={h} W={w} tcgen05={tc}: {ms:.3f} ms, "
          f"{pairs * 4 * hd / ms / 1e9:.1f} TFLOP/s; bounded-wait flag {D.ffi.lib().nlh_swa_tc_timeout_flag()}")


if __name__ == "__main__":
    case = sys.argv[1] if len(sys.argv) > 1 else "titans_level0"
    args = [int(a) for a in sys.argv[2:]]
    {"titans_level0": titans_level0, "swa_forward": swa_forward}[case](*args)
