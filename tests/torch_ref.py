"""Plain PyTorch (autograd) statements of the hot-path operators, used by tests as the
reference for the model-level harness: the memory recurrences as token loops and SWA as a
masked softmax. Same call signatures as nl_hecate_b200.stacked_mag.titans_memory / swa."""
import math

import torch


def titans_memory_ref(k, v, q, alpha, theta, eta, m0, chunk):
    n, s, d = k.shape
    M = m0.view(n, d, d).clone()
    S = torch.zeros_like(M)
    M0 = M
    ys = []
    for t in range(s):
        if chunk and t % chunk == 0:
            M0 = M
        src = M0 if chunk else M
        e = torch.einsum("nij,nj->ni", src, k[:, t]) - v[:, t]
        S = eta[:, t, None, None] * S - theta[:, t, None, None] * e[:, :, None] * k[:, t, None, :]
        M = (1 - alpha[:, t, None, None]) * M + S
        ys.append(torch.einsum("nij,nj->ni", M, q[:, t]))
    return torch.stack(ys, 1), M.reshape(n, d * d).detach()


def swa_ref(q, k, v, num_heads, head_dim, window):
    b, s, _ = q.shape
    sh = lambda t: t.float().view(b, s, num_heads, head_dim).permute(0, 2, 1, 3)
    qh, kh, vh = sh(q), sh(k), sh(v)
    sc = qh @ kh.transpose(-1, -2) / math.sqrt(head_dim)
    i = torch.arange(s, device=q.device)
    ok = (i[None, :] <= i[:, None]) & (i[None, :] >= i[:, None] + 1 - window)
    sc = sc.masked_fill(~ok, float("-inf"))
    out = torch.softmax(sc, -1) @ vh
    return out.permute(0, 2, 1, 3).reshape(b, s, num_heads * head_dim).to(q.dtype)
