"""Plain, slow statement of the Fivedra design in PyTorch (float64), one function per mechanism, whole sequences at once with the
recurrences as Python loops over the tokens.  It shares no code with the serving path: the GPU tests compare the engine with these
functions.

A model is a config dict (the shape of config.json) and a dict of tensors by checkpoint name.  A layer adds two branches that read the
SAME stream, each behind its own weighted RMS norm (weights stored as offsets from one): x <- x + mixer(n1(x)) + ff(n2(x)).  Mixers:
  'mingru'            an element-wise gated recurrence whose gate and candidate read only the current token;
  'parallel'          two mixers on the same input, summed with two constants: sliding-window attention whose values ARE its keys, with
                      a learned bias by bucketed distance and one extra unit in the softmax denominator, beside a matrix memory with
                      exponential input gate, sigmoid forget gate and a running maximum that keeps the exponentials bounded;
  'latent_attention'  causal attention over a cached low-rank latent and one rotated key part shared by all heads, queries through a
                      normalised latent of their own, rotation with frequency interpolation, and a learned per-head sink.
The feed-forward is down(relu(up h)^2).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the distance of the gain from one."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -(torch.clamp(-z, min=0.0) + torch.log1p(torch.exp(-z.abs())))


# ---- element-wise gated recurrence
def mingru_candidate(u: torch.Tensor) -> torch.Tensor:
    """Positive everywhere and continuous at 0: u + 1/2 on the right, the logistic function on the left."""
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, W] -> [T, W].  S_t = (1 - z_t) S_(t-1) + z_t c_t per channel, S_(-1) = 0; read out through a silu gate."""
    T = h.shape[0]
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    c = mingru_candidate(h @ w[p + "x"].T + w[p + "x.b"])
    g = silu(h @ w[p + "g"].T)
    S = torch.zeros(z.shape[1], dtype=h.dtype) if state is None else state.clone()
    rows = []
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        rows.append(S * g[t])
    return torch.stack(rows) @ w[p + "o"].T


# ---- sliding-window attention whose values are its keys
def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the bias table for distance n >= 0: one row per distance below rows // 2, then logarithmic steps that reach the last row
    at distance `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def keyvalue_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    rel = w[p + "rel"]
    rows, span = rel.shape[0], m["mask"]["size"]
    idx = torch.tensor([[distance_bucket(i - j, rows, m["bias_max"]) if i >= j else 0 for j in range(T)] for i in range(T)])
    i_, j_ = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j_ <= i_) & (i_ - j_ < span)
    out = torch.zeros(T, H, d, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] + rel[:, hd][idx]
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        top = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        pr = e / (torch.exp(-top) + e.sum(-1, keepdim=True))        # the extra unit: a key of score 0 without a value
        out[:, hd] = pr @ k[:, g]
    return out.reshape(T, H * d) @ w[p + "o"].T


# ---- matrix memory with exponential gating
def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def matrix_memory(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    li = capped(h @ w[p + "i"].T + w[p + "i.b"], cap)                       # log of the input gate
    lf = log_sigmoid(capped(h @ w[p + "f"].T + w[p + "f.b"], cap))          # log of the forget gate
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        n = torch.zeros(d, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)                                # running maximum: starts at 0
        for t in range(T):
            new = torch.maximum(lf[t, hd] + mx, li[t, hd])
            keep, put = torch.exp(lf[t, hd] + mx - new), torch.exp(li[t, hd] - new)
            S = keep * S + put * torch.outer(k[t, hd], v[t, hd])
            n = keep * n + put * k[t, hd]
            mx = new
            den = torch.maximum((n @ q[t, hd]).abs(), torch.exp(-mx)) + 1e-6
            o[t, hd] = (S.T @ q[t, hd]) / den
    o = rms_unit(o, eps).reshape(T, H * dv) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float) -> torch.Tensor:
    return m["left_scale"] * keyvalue_attention(h, w, p + "left.", m["left"]) + m["right_scale"] * matrix_memory(h, w, p + "right.", m["right"], eps)


# ---- latent attention
def rotary_frequencies(rot: Dict) -> (torch.Tensor, float):
    """Per-pair frequencies and the common factor on cos / sin.  Without 'scaling': base^(-2i / dims) and 1.  With it, pairs whose
    wavelength is long against the original context are slowed by `factor`, short ones are kept, with a linear ramp between."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=DT)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor = float(sc["factor"])

    def turn_index(turns: float) -> float:          # the (fractional) pair whose wavelength makes `turns` turns over the original context
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_index(sc["fast"])), 0)
    hi = min(math.ceil(turn_index(sc["slow"])), dims - 1)
    ramp = torch.clamp((torch.arange(dims // 2, dtype=DT) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: torch.Tensor, pos: torch.Tensor, rot: Dict) -> torch.Tensor:
    """x [T, ..., r]: entries (2i, 2i + 1), i < dims / 2, turned by pos * f_i; the rest unchanged."""
    f, mag = rotary_frequencies(rot)
    dims = int(rot["dims"])
    a = pos.to(DT)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(a) * mag).view(shape), (torch.sin(a) * mag).view(shape)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict, eps: float, pos0: int = 0) -> torch.Tensor:
    T = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(pos0, pos0 + T)
    cq = rms_unit(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, d + r)
    qu, qr = q[..., :d], rotate_interleaved(q[..., d:], pos, m["rot"])
    dkv = h @ w[p + "dkv"].T
    c = rms_unit(dkv[:, :R], eps) * w[p + "dkv.norm"]
    kr = rotate_interleaved(dkv[:, R:], pos, m["rot"])                      # one rotated key part for all heads
    ku = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    i_, j_ = torch.arange(T)[:, None], torch.arange(T)[None, :]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        s = (qu[:, hd] @ ku[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        s = torch.where(j_ <= i_, s, torch.full_like(s, -math.inf))
        sink = w[p + "sink"][hd]
        top = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        pr = e / (torch.exp(sink - top) + e.sum(-1, keepdim=True))          # the sink takes weight and gives nothing
        out[:, hd] = pr @ v[:, hd]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ---- feed-forward, layer, model
def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, L: Dict, eps: float) -> torch.Tensor:
    kind, m = L["type"], L["mixer"]
    if kind == "mingru":
        return mingru(h, w, p)
    if kind == "parallel":
        return parallel_mixer(h, w, p, m, eps)
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps)
    raise ValueError(kind)


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, L: Dict, eps: float) -> torch.Tensor:
    p = f"l{i}."
    y = mixer(offset_norm(x, w[p + "norm1"], eps), w, p + "mix.", L, eps)
    if L.get("mlp"):
        y = y + dense_ff(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
    return x + y


def forward(cfg: Dict, w: Dict[str, torch.Tensor], tokens: List[int], taps: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """-> logits [T, vocab]; taps (optional list) receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    for i, L in enumerate(cfg["layers"]):
        x = layer(x, w, i, L, eps)
        if taps is not None:
            taps.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T


MIXERS = {
    "mingru": lambda h, w, p, m, eps: mingru(h, w, p),
    "parallel": parallel_mixer,
    "latent_attention": latent_attention,
}


def random_weights(cfg: Dict, seed: int = 0, sizes: Optional[Dict[int, Dict[str, int]]] = None) -> Dict[str, torch.Tensor]:
    """Random tensors with the checkpoint's names and shapes, values representable in bfloat16.  `sizes[layer]['rel_rows']` is the row
    count of a 'parallel' layer's distance-bias table (config.json leaves it to the tensor's shape)."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out: Dict[str, torch.Tensor] = {}
    sizes = sizes or {}

    def mat(name, o, i, s=None):
        out[name] = (torch.randn(o, i, generator=g) * (s if s is not None else 1.0 / math.sqrt(i))).bfloat16().float()

    def vec(name, n, s=0.1, mean=0.0):
        out[name] = (mean + torch.randn(n, generator=g) * s).bfloat16().float()

    out["embed"] = (torch.randn(V, W, generator=g) * 0.5).bfloat16().float()
    vec("final.norm", W, 0.2)
    mat("head", V, W)
    for li, L in enumerate(cfg["layers"]):
        p, m = f"l{li}.", L["mixer"]
        vec(p + "norm1", W, 0.2)
        q = p + "mix."
        if L["type"] == "mingru":
            C = m["width"]
            mat(q + "z", C, W); vec(q + "z.b", C, 0.5)
            mat(q + "x", C, W); vec(q + "x.b", C, 0.5)
            mat(q + "g", C, W); mat(q + "o", W, C)
        elif L["type"] == "parallel":
            a, ql = m["left"], q + "left."
            H, G, d = a["heads"], a["kv_heads"], a["dim"]
            mat(ql + "q", H * d, W); vec(ql + "q.b", H * d, 0.3)
            mat(ql + "k", G * d, W); vec(ql + "k.b", G * d, 0.3)
            mat(ql + "rel", sizes.get(li, {}).get("rel_rows", 8), H, 1.0)
            mat(ql + "o", W, H * d)
            r, qr = m["right"], q + "right."
            H, d, dv = r["heads"], r["dim"], r["vdim"]
            mat(qr + "q", H * d, W); mat(qr + "k", H * d, W); mat(qr + "v", H * dv, W); mat(qr + "g", H * dv, W)
            mat(qr + "i", H, W, 1.5 / math.sqrt(W)); vec(qr + "i.b", H, 0.5)
            mat(qr + "f", H, W, 1.5 / math.sqrt(W)); vec(qr + "f.b", H, 0.5, 2.0)
            vec(qr + "norm", H * dv, 0.1, 1.0); mat(qr + "o", W, H * dv)
        elif L["type"] == "latent_attention":
            H, d, r, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            mat(q + "dq", Q, W); vec(q + "dq.norm", Q, 0.1, 1.0); mat(q + "uq", H * (d + r), Q)
            mat(q + "dkv", R + r, W); vec(q + "dkv.norm", R, 0.1, 1.0)
            mat(q + "uk", H * d, R); mat(q + "uv", H * dv, R)
            vec(q + "sink", H, 1.0); mat(q + "o", W, H * dv)
        else:
            raise ValueError(L["type"])
        f = L.get("mlp")
        if f is not None:
            vec(p + "norm2", W, 0.2)
            mat(p + "mlp.up", f["ff"], W); mat(p + "mlp.down", W, f["ff"])
    return out
