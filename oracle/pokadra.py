"""oracle.pokadra — the Pokadra decoder restated in plain torch on the CPU.  TEST INFRASTRUCTURE.

One function per mechanism, written from the design's equations and sharing nothing with the
product path (`scalellm_b200/`).  Everything runs in one floating-point type (float64 by default)
over an explicit per-sequence state, so the same functions serve whole prompts, portions and
single decoded tokens.

Notation (W = width, m = residual multiplier, L layers):

    x_0      = scale * E[tok] + B[(mul_prev * prev + mul_cur * tok) mod buckets]    (B[buckets] at a sequence's start)
    gnorm(y) = per group of W / groups consecutive channels: y / sqrt(mean(y^2) + eps), then * w
    layer i  : x <- x + m gnorm1(mixer(x)) ; x <- x + m gnorm2(ff(x)) ;
               x <- x + m rms(P (gelu(Gx) * e_i[tok])) * w_side             (e_i: slice i of the side table)
    history  : X_0 = x_0, X_{i+1} = result of layer i ; input of layer i+1 = sum_{j <= i+1} c_i[j] X_j
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .kigalix import read_safetensors  # noqa: F401  (same file format)

SQRT_2_OVER_PI = math.sqrt(2.0 / math.pi)
SWISH_SLOPE = 1.702           # the feed-forward's gate is g * sigmoid(1.702 g)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(SQRT_2_OVER_PI * (z + 0.044715 * z ** 3)))


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def group_norm(y: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    shape = y.shape
    return (rms(y.reshape(*shape[:-1], groups, shape[-1] // groups), eps)).reshape(shape) * w


def embedding(tokens: List[int], prev: Optional[int], w: Dict[str, torch.Tensor], emb: dict) -> torch.Tensor:
    """prev: the token before tokens[0], None at the start of the sequence."""
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(emb.get("scale", 1.0))
    bg = emb.get("bigram")
    if bg:
        n, a, b = int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])
        rows, p = [], prev
        for t in tokens:
            rows.append(n if p is None else (p * a + t * b) % n)
            p = t
        x = x + w["bigram"][torch.tensor(rows, dtype=torch.long)]
    return x


def rotary_frequencies(rot: dict) -> (torch.Tensor, float):
    """(frequency per pair [dims / 2], multiplier of cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])
    where = lambda t: dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    out = []
    for i in range(dims // 2):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(float(f[i]) / factor * r + float(f[i]) * (1.0 - r))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, pos: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, ..., dim]: pairs (2i, 2i+1) of the first rot.dims channels turn by pos * f_i."""
    if not rot:
        return x
    f, mult = rotary_frequencies(rot)
    dims = int(rot["dims"])
    ang = pos.to(torch.float64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(ang) * mult).to(x.dtype).reshape(shape), (torch.sin(ang) * mult).to(x.dtype).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(i: int, j: int, mask: Optional[dict]) -> bool:
    if j > i:
        return False
    if not mask or "size" not in mask:
        return True
    return i - j < int(mask["size"]) or j < int(mask.get("keep_first", 0))


def diff_lambda(w: Dict[str, torch.Tensor], diff: float) -> float:
    return float(torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum())) + diff


def diff_attend(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, pos: torch.Tensor, scale: float,
                mask: Optional[dict], lam: float, diff: float, eps: float) -> torch.Tensor:
    """q [T, H, 2, dim] at positions pos over keys K [n, G, 2, dim] and values V [n, G, vdim] (row j = position j):
    per head softmax(s1) V - lam softmax(s2) V, divided by its root mean square, times (1 - diff).  [T, H, vdim]"""
    T, H = q.shape[0], q.shape[1]
    G = K.shape[1]
    out = torch.zeros(T, H, V.shape[2], dtype=q.dtype)
    for t in range(T):
        i = int(pos[t])
        js = [j for j in range(i + 1) if visible(i, j, mask)]
        for hh in range(H):
            g = hh // (H // G)
            a = []
            for mp in range(2):
                s = (K[js, g, mp, :] @ q[t, hh, mp, :]) * scale
                a.append(torch.softmax(s, dim=0) @ V[js, g, :])
            out[t, hh] = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    return out


def diff_attention(h: torch.Tensor, pos: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                   kv: dict, shared: Optional[dict]) -> torch.Tensor:
    """kv: this layer's {"k": [n, G, 2, dim], "v": [n, G, vdim]} (grown here unless `shared` — another
    layer's kv, already holding this step's rows — is given)."""
    H, G, dim, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, 2, dim)
    q = rotate(rms(q, eps) * w["q.norm"], pos, m.get("rot"))
    if shared is None:
        k = (h @ w["k"].T).reshape(T, G, 2, dim)
        k = rotate(rms(k, eps) * w["k.norm"], pos, m.get("rot"))
        v = (h @ w["v"].T).reshape(T, G, vd)
        kv["k"] = torch.cat([kv["k"], k]) if "k" in kv else k
        kv["v"] = torch.cat([kv["v"], v]) if "v" in kv else v
    else:
        kv = shared
    diff = float(m["diff"])
    o = diff_attend(q, kv["k"], kv["v"], pos, float(m["scale"]), m.get("mask"), diff_lambda(w, diff), diff, eps)
    gate = torch.sigmoid(h @ w["g"].T)                     # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * vd) @ w["o"].T


def mingru(h: torch.Tensor, w: Dict[str, torch.Tensor], st: dict) -> torch.Tensor:
    z = torch.sigmoid(h @ w["z"].T + w["z.b"])
    u = h @ w["x"].T + w["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = h @ w["g"].T
    S = st.get("S", torch.zeros(z.shape[1], dtype=h.dtype))
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S * g[t] * torch.sigmoid(g[t]))
    st["S"] = S
    return torch.stack(rows) @ w["o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    lim = float(mlp["limit"])
    g = torch.clamp(h @ w["gate"].T, max=lim)
    u = torch.clamp(h @ w["up"].T, min=-lim, max=lim)
    return (g * torch.sigmoid(SWISH_SLOPE * g) * (u + 1.0)) @ w["down"].T


def token_side(x: torch.Tensor, tokens: List[int], layer: int, w: Dict[str, torch.Tensor], pre: str, dim: int,
               eps: float) -> torch.Tensor:
    """The normalised per-token term of layer `layer` (to be scaled by m and added)."""
    e = w["side.embed"][torch.tensor(tokens, dtype=torch.long)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[pre + "side.gate"].T) * e) @ w[pre + "side.proj"].T
    return rms(y, eps) * w[pre + "side.norm"]


class Pokadra:
    def __init__(self, config: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float64):
        self.cfg, self.dtype = config, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.groups = int(config["norm"].get("groups", 1))
        self.m = float(config.get("residual_mult", 1.0))

    def sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        n = len(prefix)
        return {k[n:]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self) -> dict:
        return {"layers": [dict() for _ in self.cfg["layers"]], "n": 0, "prev": None}

    def forward(self, tokens: List[int], state: dict, layer_out: Optional[list] = None) -> torch.Tensor:
        """Runs the next tokens of one sequence; returns logits [T, vocab]."""
        w, eps, m = self.w, self.eps, self.m
        T = len(tokens)
        pos = torch.arange(state["n"], state["n"] + T)
        x = embedding(tokens, state["prev"], w, self.cfg.get("embedding", {})).to(self.dtype)
        state["n"] += T
        state["prev"] = tokens[-1]
        hist = [x]
        for i, L in enumerate(self.cfg["layers"]):
            st, p = state["layers"][i], f"l{i}."
            mw = self.sub(p + "mix.")
            if L["type"] == "attention":
                src = L["mixer"].get("kv_from")
                y = diff_attention(x, pos, mw, L["mixer"], eps, st, None if src is None else state["layers"][int(src)])
            elif L["type"] == "mingru":
                y = mingru(x, mw, st)
            else:
                raise ValueError(L["type"])
            x = x + m * group_norm(y, w[p + "norm1"], self.groups, eps)
            if L.get("mlp") is not None:
                x = x + m * group_norm(dense_ff(x, self.sub(p + "mlp."), L["mlp"]), w[p + "norm2"], self.groups, eps)
            if self.cfg.get("token_side"):
                x = x + m * token_side(x, tokens, i, w, p, int(self.cfg["token_side"]["dim"]), eps)
            hist.append(x)
            if p + "dwa" in w:
                x = sum(w[p + "dwa"][j] * hist[j] for j in range(i + 2))
            if layer_out is not None:
                layer_out.append(x)
        return group_norm(x, w["final.norm"], self.groups, eps) @ w["head"].T
