"""oracle.kigalix — the Kigalix decoder restated in plain torch on the CPU.  TEST INFRASTRUCTURE.

One function per mechanism, written from the design's equations and sharing nothing with the
product path (`scalellm_b200/`).  Everything runs in one floating-point type (float64 by default)
token by token or chunk by chunk over an explicit per-sequence state, so that the same functions
serve as the oracle for whole prompts, for portions and for single decoded tokens.

Notation used below (W = width, S = number of residual streams):

    norm(x; w)       = x / sqrt(mean(x^2) + eps) * (1 + w)               "offset" RMS norm
    plain_norm(x; w) = x / sqrt(mean(x^2) + eps) * w
    shift(n_t)       = n_t + (n_{t-1} - n_t) * mu          (n_{-1} = 0; n_{t-1} is unshifted)
    sublayer q of a layer, streams X = (x_1 .. x_S):
        u = sum_s in_q[s] x_s ;  n = norm(u)
        y = f_q(shift(n) for the mixer, n for the feed-forward) * sigmoid(G_q n + b_q)
        x_t' = sum_s mix_q[s, t] x_s + out_q[t] y
"""
from __future__ import annotations

import json
import math
import struct
from typing import Dict, List, Optional

import numpy as np
import torch

SQRT_2_OVER_PI = math.sqrt(2.0 / math.pi)
DELTA_DECAY_SCALE = math.exp(-0.5)      # w = exp(-e^{-1/2} * sigmoid(.))
UNIT_KEY_EPS = 1e-6


# --------------------------------------------------------------------------- checkpoint reading
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, raw data."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = np.frombuffer(raw, dtype=np.uint8, count=hi - lo, offset=base + lo).copy()
        dt = meta["dtype"]
        if dt == "BF16":
            t = torch.from_numpy(buf.view(np.int16)).view(torch.bfloat16)
        elif dt == "F32":
            t = torch.from_numpy(buf.view(np.float32))
        elif dt == "F16":
            t = torch.from_numpy(buf.view(np.float16))
        elif dt == "I32":
            t = torch.from_numpy(buf.view(np.int32))
        elif dt == "I64":
            t = torch.from_numpy(buf.view(np.int64))
        else:
            raise ValueError(f"dtype {dt} of {name}")
        out[name] = t.reshape(meta["shape"])
    return out


# --------------------------------------------------------------------------- small mechanisms
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def plain_norm(x, w, eps):
    return rms_unit(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(SQRT_2_OVER_PI * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def token_shift(n: torch.Tensor, prev: torch.Tensor, mu: torch.Tensor):
    """n [T, W] (unshifted), prev [W] = the last unshifted row of the previous portion (zeros at the
    start of a sequence).  Returns (shifted rows, new prev)."""
    before = torch.cat([prev[None, :], n[:-1]], dim=0)
    return n + (before - n) * mu, n[-1].clone()


def rope_table(rot: dict, dtype=torch.float64):
    """Per-pair angular frequencies and the cos/sin multiplier of one rotary configuration."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def corr(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(corr(float(sc["fast"]))), 0)
        hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return f, mult


def rope_interleaved(x: torch.Tensor, pos: torch.Tensor, f: torch.Tensor, mult: float) -> torch.Tensor:
    """x [T, ..., D]; the first 2*len(f) entries of the last axis rotate pairwise (2i, 2i+1)."""
    d = 2 * f.numel()
    ang = pos.to(f.dtype)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [f.numel()]
    c, s = (torch.cos(ang) * mult).reshape(shape), (torch.sin(ang) * mult).reshape(shape)
    a, b = x[..., 0:d:2], x[..., 1:d:2]
    out = x.clone()
    out[..., 0:d:2] = a * c - b * s
    out[..., 1:d:2] = b * c + a * s
    return out


# --------------------------------------------------------------------------- mixers
def latent_attention(h: torch.Tensor, pos: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict,
                     eps: float, cache: dict) -> torch.Tensor:
    """Latent (compressed key/value) attention over the cached latents plus this portion.
    cache: {"c": [n, kv_rank], "kr": [n, rot_dim]} of the earlier tokens (grown here)."""
    H, dim, rd, vd, rank = (int(cfg[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    T = h.shape[0]
    f, mult = rope_table(cfg["rot"], h.dtype)
    q = (h @ w["q"].T).reshape(T, H, dim + rd)
    q_u, q_r = q[..., :dim], rope_interleaved(q[..., dim:], pos, f, mult)
    dkv = h @ w["dkv"].T
    c = plain_norm(dkv[:, :rank], w["dkv.norm"], eps)
    kr = rope_interleaved(dkv[:, rank:], pos, f, mult)
    cache["c"] = torch.cat([cache["c"], c], dim=0) if "c" in cache else c
    cache["kr"] = torch.cat([cache["kr"], kr], dim=0) if "kr" in cache else kr
    C, KR = cache["c"], cache["kr"]
    n = C.shape[0]
    k_u = (C @ w["uk"].T).reshape(n, H, dim)
    v = (C @ w["uv"].T).reshape(n, H, vd)
    s = (torch.einsum("thd,nhd->htn", q_u, k_u) + torch.einsum("thd,nd->htn", q_r, KR)) * float(cfg["scale"])
    key_pos = torch.arange(n)
    visible = key_pos[None, :] <= pos[:, None]
    s = s.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("htn,nhd->thd", p, v).reshape(T, H * vd)
    if "g" in w:
        o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def general_delta(h: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict, eps: float,
                  state: dict) -> torch.Tensor:
    """Generalised delta rule, one token at a time.  state["S"]: [H, dim(key), dim(value)]."""
    H, d = int(cfg["heads"]), int(cfg["dim"])
    T = h.shape[0]
    r = (h @ w["r"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, H, d)
    v = (h @ w["v"].T).reshape(T, H, d)
    decay = torch.exp(-DELTA_DECAY_SCALE * torch.sigmoid(torch.tanh(h @ w["w1"].T) @ w["w2"].T + w["w0"]))
    decay = decay.reshape(T, H, d)
    a = torch.sigmoid(h @ w["a"].T + w["a.b"]).reshape(T, H, d)
    S = state.get("S")
    if S is None:
        S = torch.zeros(H, d, d, dtype=h.dtype)
    outs = []
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(-1, keepdim=True) + UNIT_KEY_EPS)      # [H, d]
        uS = torch.einsum("hk,hkv->hv", u, S)
        S = decay[t][:, :, None] * S - (a[t] * u)[:, :, None] * uS[:, None, :] \
            + k[t][:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hkv,hk->hv", S, r[t]))
    state["S"] = S
    o = torch.stack(outs, 0)                               # [T, H, d]
    o = rms_unit(o, eps).reshape(T, H * d) * w["norm"]
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# --------------------------------------------------------------------------- feed-forward
def dense_ff(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def moe_ff(h, w, cfg):
    E, top = int(cfg["router"]["experts"]), int(cfg["router"]["top"])
    s = torch.sigmoid(h.to(torch.float32).to(h.dtype) @ w["router"].T)
    val, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for e in range(E):
        for j in range(top):
            rows = (idx[:, j] == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            x = h[rows] * val[rows, j][:, None]
            out[rows] += (silu(x @ w[f"e{e}.gate"].T) * (x @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T
    return out


# --------------------------------------------------------------------------- model
class Kigalix:
    def __init__(self, config: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float64):
        self.cfg, self.dtype = config, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.S = int(config.get("streams", 1))

    def sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        n = len(prefix)
        return {k[n:]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self) -> dict:
        return {"layers": [dict() for _ in self.cfg["layers"]], "n": 0}

    def forward(self, tokens: List[int], state: dict, layer_out: Optional[list] = None) -> torch.Tensor:
        """Runs the next tokens of one sequence; returns logits [T, vocab]."""
        w, eps = self.w, self.eps
        T = len(tokens)
        pos = torch.arange(state["n"], state["n"] + T)
        state["n"] += T
        x0 = w["embed"][torch.tensor(tokens, dtype=torch.long)]
        X = [x0.clone() for _ in range(self.S)]
        for i, L in enumerate(self.cfg["layers"]):
            st = state["layers"][i]
            p = f"l{i}."
            for q in (1, 2):
                if q == 2 and L.get("mlp") is None:
                    continue
                hc = {k: w[f"{p}hc{q}.{k}"] for k in ("in", "out", "mix")}
                u = sum(hc["in"][s] * X[s] for s in range(self.S))
                n = offset_norm(u, w[f"{p}norm{q}"], eps)
                if q == 1:
                    hs, st["prev"] = token_shift(n, st.get("prev", torch.zeros_like(n[0])), w[p + "shift"])
                    mw = self.sub(p + "mix.")
                    if L["type"].startswith("latent_attention"):
                        y = latent_attention(hs, pos, mw, L["mixer"], eps, st.setdefault("kv", {}))
                    elif L["type"] == "general_delta":
                        y = general_delta(hs, mw, L["mixer"], eps, st)
                    else:
                        raise ValueError(L["type"])
                else:
                    fw = self.sub(p + "mlp.")
                    y = dense_ff(n, fw) if L["mlp"]["kind"] == "dense" else moe_ff(n, fw, L["mlp"])
                y = y * torch.sigmoid(n @ w[f"{p}rg{q}"].T + w[f"{p}rg{q}.b"])
                X = [sum(hc["mix"][s, t] * X[s] for s in range(self.S)) + hc["out"][t] * y
                     for t in range(self.S)]
            if layer_out is not None:
                layer_out.append(sum(X))
        x = offset_norm(sum(X), w["final.norm"], eps)
        return x @ w["head"].T
