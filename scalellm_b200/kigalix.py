"""Kigalix: a decoder-only model whose layers are listed in its config.json.

    x_1 .. x_S = embed[token]                         S fp32 residual streams (config "streams")
    per layer  : mixer sublayer, then (unless "mlp" is null) a feed-forward sublayer, each read from
                 and written to the streams through a HyperConnection (offset RMS norm, gated result);
                 the mixer reads the token-shifted rows.
    mixers     : "latent_attention" / "latent_attention_2" (layers.LatentAttention; the second kind has
                 YaRN-scaled rotary frequencies from "rot.scaling" and an output gate),
                 "general_delta" (layers.DeltaRuleMixer)
    feed-forward: "dense" (GELU-tanh gated MLP) or "moe" (sigmoid-routed SiLU experts, layers.SparseMoE)
    output     : offset RMS norm of the sum of the streams, then the vocabulary projection.

Every size and constant is read from config.json or a tensor's shape.  Tensor names: "embed", "head",
"final.norm", and per layer i "l<i>.norm1|norm2", "l<i>.shift", "l<i>.rg1|rg2(.b)", "l<i>.hc1|hc2.in|out|mix",
"l<i>.mix.*", "l<i>.mlp.*" (experts "e<j>.gate|up|down", "router").

State per sequence: the last normalised row of every layer (token shift) and the delta-rule matrices
live in state slots; latents and rotary keys of the attention layers in paged LatentKVCache rows.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from . import _lib, kernels
from .layers import (DeltaRuleMixer, GatedMLP, HyperConnection, InputParameters, LatentAttention,
                     LatentKVCache, Linear, SparseMoE, TokenShift, apply_yarn_rope_scaling)
from .registry import register_model

# constants the design fixes
DELTA_DECAY_SCALE = math.exp(-0.5)     # decay = exp(-e^{-1/2} sigmoid(.))
DELTA_KEY_EPS = 1e-6                   # under the root of the unit key
NORM_OFFSET = 1.0                      # layer norms store their weight around zero


def rotary_table(rot: dict):
    """(inv_freq [dims / 2] fp32, multiplier of cos and sin) of a layer's "rot" entry."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        return apply_yarn_rope_scaling(inv_freq, base, dims, float(sc["factor"]), float(sc["original"]),
                                       float(sc["fast"]), float(sc["slow"]))
    return inv_freq.to(torch.float32), 1.0


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    """Names and shapes of a checkpoint of this config."""
    W, V, S = int(config["width"]), int(config["vocab"]), int(config.get("streams", 1))
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(config["layers"]):
        p, m = f"l{i}.", L["mixer"]
        subs = (1, 2) if L.get("mlp") is not None else (1,)
        for q in subs:
            out[f"{p}norm{q}"] = (W,)
            out[f"{p}rg{q}"] = (W, W)
            out[f"{p}rg{q}.b"] = (W,)
            out[f"{p}hc{q}.in"] = (S,)
            out[f"{p}hc{q}.out"] = (S,)
            out[f"{p}hc{q}.mix"] = (S, S)
        out[p + "shift"] = (W,)
        if L["type"].startswith("latent_attention"):
            H, dim, rd, vd, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
            out.update({p + "mix.q": (H * (dim + rd), W), p + "mix.dkv": (rank + rd, W),
                        p + "mix.dkv.norm": (rank,), p + "mix.uk": (H * dim, rank),
                        p + "mix.uv": (H * vd, rank), p + "mix.o": (W, H * vd)})
            if L["type"] == "latent_attention_2":
                out[p + "mix.g"] = (H * vd, W)
        elif L["type"] == "general_delta":
            n = int(m["heads"]) * int(m["dim"])
            lr = int(m.get("decay_rank", 16))   # a checkpoint fixes it by the shape of w1 / w2
            out.update({p + f"mix.{k}": (n, W) for k in ("r", "k", "v", "g", "a")})
            out.update({p + "mix.a.b": (n,), p + "mix.w1": (lr, W), p + "mix.w2": (n, lr), p + "mix.w0": (n,),
                        p + "mix.norm": (n,), p + "mix.o": (W, n)})
        else:
            raise ValueError(f"unknown mixer type {L['type']!r}")
        mlp = L.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            out.update({p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
        elif mlp["kind"] == "moe":
            ff, E = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
            out[p + "mlp.router"] = (E, W)
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
        else:
            raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
    return out


def random_tensors(config: dict, seed: int = 0, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights of the architecture (bench and tests): projections N(0, 1/in), small vectors."""
    g = torch.Generator().manual_seed(seed)
    S = int(config.get("streams", 1))
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if name.endswith("hc1.mix") or name.endswith("hc2.mix"):
            t = torch.eye(S) + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "in" and ".hc" in name:
            t = torch.full(shape, 1.0 / S) + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "out" and ".hc" in name:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "shift":
            t = torch.rand(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.2 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


class _Layer:
    hc1: HyperConnection
    hc2: Optional[HyperConnection] = None
    shift: Optional[TokenShift] = None
    mixer = None
    ff = None
    kind: str = ""
    cache: Optional[LatentKVCache] = None


@register_model("Kigalix")
class KigalixDecoder:
    needs_state_slots = True
    CSRC = ("hyper.cu", "latent_attn.cu", "delta_rule.cu", "moe.cu")

    def __init__(self, config: dict, dtype: torch.dtype, device, max_seqs: int = 4):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Kigalix runs in bfloat16 or float32")
        _lib.ensure(self.CSRC)
        self.config, self.dtype, self.device, self.max_seqs = config, dtype, torch.device(device), max_seqs
        self.width, self.n_vocab = int(config["width"]), int(config["vocab"])
        self.n_streams = int(config.get("streams", 1))
        self.eps = float(config["norm"]["eps"])
        self.layers: List[_Layer] = []
        self.embed = self.final_norm = self.head = None

    @classmethod
    def from_config(cls, config: dict, dtype, device, max_seqs: int = 4) -> "KigalixDecoder":
        return cls(config, dtype, device, max_seqs)

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0) -> None:
        self.load_weights(random_tensors(self.config, seed))

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        dev, dt, eps = self.device, self.dtype, self.eps
        missing = [n for n in tensor_shapes(self.config) if n not in tensors]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        w = lambda name: tensors[name].to(dev).to(dt)
        opt = lambda name: tensors[name].to(dev) if name in tensors else None
        self.embed = w("embed").contiguous()
        self.final_norm = tensors["final.norm"].to(dev).to(torch.float32).contiguous()
        self.head = Linear(w("head"))
        self.layers = []
        for i, L in enumerate(self.config["layers"]):
            p, m = f"l{i}.", L["mixer"]
            lay = _Layer()
            lay.kind = L["type"]

            def hyper(q: int) -> HyperConnection:
                gate = Linear(w(f"{p}rg{q}")) if f"{p}rg{q}" in tensors else None
                return HyperConnection(tensors[f"{p}norm{q}"].to(dev), eps, NORM_OFFSET, opt(f"{p}hc{q}.in"),
                                       opt(f"{p}hc{q}.mix"), opt(f"{p}hc{q}.out"), gate, opt(f"{p}rg{q}.b"), dt)
            lay.hc1 = hyper(1)
            if p + "shift" in tensors:
                lay.shift = TokenShift(tensors[p + "shift"].to(dev), self.max_seqs, dt, dev)
            mw = {k[len(p) + 4:]: w(k) for k in tensors if k.startswith(p + "mix.")}
            if L["type"].startswith("latent_attention"):
                inv_freq, mult = rotary_table(m["rot"])
                lay.mixer = LatentAttention(mw, int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]),
                                            int(m["kv_rank"]), float(m["scale"]), inv_freq, mult,
                                            int(m["rot"]["dims"]), eps, dt, dev)
            elif L["type"] == "general_delta":
                lay.mixer = DeltaRuleMixer(mw, int(m["heads"]), int(m["dim"]), DELTA_DECAY_SCALE, DELTA_KEY_EPS, eps,
                                           self.max_seqs, dt, dev)
            else:
                raise ValueError(f"unknown mixer type {L['type']!r}")
            mlp = L.get("mlp")
            if mlp is not None:
                lay.hc2 = hyper(2)
                f = p + "mlp."
                if mlp["kind"] == "dense":
                    lay.ff = GatedMLP(w(f + "gate"), w(f + "up"), w(f + "down"), "gelu_tanh")
                elif mlp["kind"] == "moe":
                    E = int(mlp["router"]["experts"])
                    stack = lambda leaf: torch.stack([w(f"{f}e{e}.{leaf}") for e in range(E)], dim=0)
                    lay.ff = SparseMoE(tensors[f + "router"].to(dev), stack("gate"), stack("up"), stack("down"),
                                       int(mlp["router"]["top"]), "silu")
                else:
                    raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
            self.layers.append(lay)

    # ------------------------------------------------------------------ cache
    def alloc_cache(self, n_blocks: int, block_size: int) -> None:
        for lay, L in zip(self.layers, self.config["layers"]):
            if L["type"].startswith("latent_attention"):
                m = L["mixer"]
                lay.cache = LatentKVCache(n_blocks, block_size, int(m["kv_rank"]), int(m["rot_dim"]), self.dtype,
                                          self.device)

    # ------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, params: InputParameters,
                last_token_idxes: Optional[torch.Tensor] = None, layer_out: Optional[list] = None) -> torch.Tensor:
        """One step over the packed rows of all sequences; logits [rows or len(last_token_idxes), vocab].
        layer_out, if given, receives the sum of the streams after every layer (fp32)."""
        X = kernels.embed_streams(self.embed, tokens, self.n_streams)
        for lay in self.layers:
            n, n32 = lay.hc1.read(X, want_fp32=True)
            hs = lay.shift(n32, positions, params) if lay.shift is not None else n
            if lay.cache is not None:
                y = lay.mixer(hs, positions, lay.cache, params)
            else:
                y = lay.mixer(hs, positions, params)
            lay.hc1.write(X, y, n)
            if lay.ff is not None:
                n2 = lay.hc2.read(X)
                lay.hc2.write(X, lay.ff(n2), n2)
            if layer_out is not None:
                layer_out.append(X.sum(dim=1))
        if last_token_idxes is not None:
            X = X.index_select(0, last_token_idxes.to(torch.int64))
        hn = kernels.hc_norm(X, None, self.final_norm, self.eps, NORM_OFFSET, self.dtype)
        return self.head(hn)

    __call__ = forward
