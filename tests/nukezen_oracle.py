"""Plain, slow statement of the Nukezen design in PyTorch (float64 by default), one function per mechanism, whole sequences at once or
token by token in Python loops.  It shares no code with the serving path: the GPU tests compare the engine with these functions.

A model is a config dict (the shape of config.json) and a dict of tensors by checkpoint name.  Layers come in three kinds:
  'parallel'       two mixers on the same input, summed with two constants: windowed rotary softmax attention with an element-wise
                   sigmoid output gate, and a state-space recurrence with scalar decay per head (short convolution in front, gated
                   grouped norm behind);
  'channel_delta'  a delta-rule recurrence whose decay has one factor per head and key channel;
  'attention'      chunk-local attention without rotation: tanh-capped scores, a learned bias by bucketed distance, and a softmax whose
                   denominator carries an extra one.
Every sublayer reads the stream itself; its output is RMS-normalised with a weight vector and added.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, H, d]: entries (2i, 2i + 1), i < dims / 2, turned by the angle pos * base^(-2i / dims); the rest unchanged."""
    out = x.clone()
    for i in range(dims // 2):
        a = pos.to(DT) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def short_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], w [C, taps]: y_t = sum_j w[:, j] * x_(t - taps + 1 + j), zeros before the sequence."""
    T, C = x.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    if bias is not None:
        y = y + bias
    return y


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """The attention half of a 'parallel' mixer.  h [T, W] -> [T, W]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q = rms_unit(q, eps) * w[p + "q.norm"]
    k = rms_unit(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    q = rotate_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"])
    span = m["mask"]["size"]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        i, j = pos[:, None], pos[None, :]
        s = s.masked_fill(~((j <= i) & (i - j < span)), float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, g]
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def state_space(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """The recurrent half of a 'parallel' mixer: S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t, token by token."""
    T = h.shape[0]
    H, P, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    S = torch.zeros(H, N, P, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.view(T, ng, inner // ng), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return m["left_scale"] * window_attention(h, w, p + "left.", m["left"], eps) + m["right_scale"] * state_space(h, w, p + "right.", m["right"], eps)


def channel_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    """Delta rule with a decay factor per head and key channel.  Per token: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, Hk, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, Hk, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, Hk, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a).view(T, H, d))
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            kh = hd // (H // Hk)
            S[hd] = g[t, hd][:, None] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, kh])
            S[hd] = S[hd] + torch.outer(k[t, kh], u)
            o[t, hd] = S[hd].T @ q[t, kh]
    o = rms_unit(o, eps) * w[p + "norm"]
    o = o.reshape(T, H * dv) * torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T)
    return o @ w[p + "o"].T


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the bias table for distance n: exact below rows // 2, then logarithmic steps that reach the last row at distance `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def chunk_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (rms_unit(h @ w[p + "q"].T, eps) * w[p + "q.norm"]).view(T, H, d)
    k = (rms_unit(h @ w[p + "k"].T, eps) * w[p + "k.norm"]).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    rel = w[p + "rel"]
    rows, cap, chunk = rel.shape[0], m["softcap"], m["mask"]["size"]
    pos = torch.arange(T)
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i) & ((i // chunk) == (j // chunk))
    bucket = torch.tensor([[distance_bucket(int(a - b), rows, m["bias_max"]) if a >= b else 0 for b in range(T)] for a in range(T)])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = cap * torch.tanh(s / cap) + rel[:, hd][bucket]
        e = torch.exp(s).masked_fill(~seen, 0.0)
        out[:, hd] = (e / (1.0 + e.sum(-1, keepdim=True))) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


MIXERS = {"parallel": parallel_mixer, "channel_delta": channel_delta, "attention": chunk_attention}


def forward(cfg: Dict, weights: Dict[str, torch.Tensor], tokens, streams: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """-> logits [T, vocab]; `streams` (optional list) receives the residual stream after every layer."""
    w = {k: v.to(DT) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    for li, L in enumerate(cfg["layers"]):
        p = f"l{L.get('weights_of', li)}."
        x = x + rms_unit(MIXERS[L["type"]](x, w, p + "mix.", L["mixer"], eps), eps) * w[p + "norm1"]
        if L.get("mlp") is not None:
            x = x + rms_unit(dense_ff(x, w, p + "mlp."), eps) * w[p + "norm2"]
        if streams is not None:
            streams.append(x.clone())
    x = rms_unit(x, eps) * w["final.norm"]
    return x @ w["embed"].T


def random_weights(cfg: Dict, seed: int = 0, sizes: Optional[Dict[int, Dict[str, int]]] = None) -> Dict[str, torch.Tensor]:
    """Random tensors with the checkpoint's names and shapes, values representable in bfloat16.  `sizes[layer]` gives what config.json
    leaves to the tensor shapes: 'rank_a' / 'rank_g' (two-matrix projections of a 'channel_delta' layer) and 'rel_rows' (bias table of an
    'attention' layer)."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out: Dict[str, torch.Tensor] = {}
    sizes = sizes or {}

    def mat(name, o, i, s=None):
        out[name] = (torch.randn(o, i, generator=g) * (s if s is not None else 1.0 / math.sqrt(i))).bfloat16().float()

    def vec(name, n, s=0.1, mean=0.0):
        out[name] = (mean + torch.randn(n, generator=g) * s).bfloat16().float()

    out["embed"] = (torch.randn(V, W, generator=g) * 0.5).bfloat16().float()
    vec("final.norm", W, 0.1, 1.0)
    for li, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p, m, sz = f"l{li}.", L["mixer"], sizes.get(li, {})
        vec(p + "norm1", W, 0.1, 1.0)
        if L["type"] == "parallel":
            a, q = m["left"], p + "mix.left."
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            mat(q + "q", H * d, W); vec(q + "q.b", H * d)
            mat(q + "k", G * d, W); vec(q + "k.b", G * d)
            mat(q + "v", G * dv, W); vec(q + "v.b", G * dv)
            vec(q + "q.norm", d, 0.2, 1.0); vec(q + "k.norm", d, 0.2, 1.0)
            mat(q + "g", H * dv, W); mat(q + "o", W, H * dv)
            r, q = m["right"], p + "mix.right."
            H, P, N, Gr = r["heads"], r["vdim"], r["state"], r["groups"]
            C = H * P + 2 * Gr * N
            mat(q + "in", 2 * H * P + 2 * Gr * N + H, W)
            mat(q + "conv", C, r["conv"], 0.5); vec(q + "conv.b", C)
            vec(q + "dt_bias", H, 0.5); vec(q + "A_log", H, 0.5); vec(q + "D", H, 0.5)
            vec(q + "norm", H * P, 0.1, 1.0); mat(q + "o", W, H * P)
        elif L["type"] == "channel_delta":
            q = p + "mix."
            H, Hk, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            ra, rg = sz.get("rank_a", 5), sz.get("rank_g", 6)
            for nm, rows in (("q", Hk * d), ("k", Hk * d), ("v", H * dv)):
                mat(q + nm, rows, W); mat(q + nm + ".conv", rows, m["conv"], 0.5)
            mat(q + "b", H, W)
            vec(q + "A_log", H, 0.5); vec(q + "norm", dv, 0.1, 1.0)
            mat(q + "a1", ra, W); mat(q + "a2", H * d, ra, 1.0); vec(q + "dt_bias", H * d, 0.5)
            mat(q + "g1", rg, W); mat(q + "g2", H * dv, rg, 1.0)
            mat(q + "o", W, H * dv)
        elif L["type"] == "attention":
            q = p + "mix."
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(q + "q", H * d, W); mat(q + "k", G * d, W); mat(q + "v", G * dv, W)
            vec(q + "q.norm", H * d, 0.2, 1.0); vec(q + "k.norm", G * d, 0.2, 1.0)
            mat(q + "rel", sz.get("rel_rows", 8), H, 1.0)
            mat(q + "o", W, H * dv)
        else:
            raise ValueError(L["type"])
        f = L.get("mlp")
        if f is not None:
            vec(p + "norm2", W, 0.1, 1.0)
            mat(p + "mlp.gate", f["ff"], W); mat(p + "mlp.up", f["ff"], W); mat(p + "mlp.down", W, f["ff"])
    return out
