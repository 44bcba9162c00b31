"""Pokadra: a decoder-only model whose layers are listed in its config.json.

    x_0        = scale * embed[tok] + bigram[(mul_prev * prev + mul_cur * tok) mod buckets]     (fp32 residual;
                 the table's last row stands in where a sequence starts)
    per layer  : x <- x + m gnorm1(mixer(x)) ; x <- x + m gnorm2(ff(x)) (unless "mlp" is null) ;
                 x <- x + m rms(P_i (gelu_tanh(G_i x) * side[tok, i-th slice])) * w_i          (config "token_side")
                 the sublayers read x itself and their RESULT is normalised (layers.PostNormResidual,
                 "norm.groups" root mean squares per row)
    history    : X_0 = x_0, X_{i+1} = the result of layer i; layer i + 1 (and, after the last layer, the output)
                 reads sum_j dwa_i[j] X_j
    mixers     : "attention" (layers.DiffAttention: differential attention, sliding window that keeps the first
                 tokens, YaRN-scaled partial rotary turn, per-head output gate, optionally over an earlier layer's
                 keys and values: "kv_from"), "mingru" (layers.MinGRUMixer)
    feed-forward: "dense" (layers.ClampedGLU)
    output     : the grouped RMS norm with "final.norm", then the vocabulary projection.

Every size and constant is read from config.json or a tensor's shape.  Tensor names: "embed", "bigram",
"side.embed", "head", "final.norm", and per layer i "l<i>.norm1|norm2", "l<i>.dwa", "l<i>.side.gate|proj|norm",
"l<i>.mix.*", "l<i>.mlp.gate|up|down".

State per sequence: the recurrence rows of the mingru layers live in state slots, the normalised rotated keys
and the values of the attention layers in paged KVCache rows (a "kv_from" layer has none of its own), and the
last token (for the bigram row of the next one) with the engine's sequence record.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from . import _lib, kernels
from .layers import (ClampedGLU, DiffAttention, InputParameters, KVCache, Linear, MinGRUMixer, PostNormResidual,
                     TokenSideInput, apply_yarn_rope_scaling)
from .registry import register_model

# constants the design fixes
GLU_SLOPE = 1.702            # the feed-forward's gate is g * sigmoid(1.702 g)


def rotary_table(rot: Optional[dict]):
    """(inv_freq [dims / 2] fp32 or None, multiplier of cos and sin, dims) of a mixer's "rot" entry."""
    if not rot:
        return None, 1.0, 0
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        f, mult = apply_yarn_rope_scaling(inv_freq, base, dims, float(sc["factor"]), float(sc["original"]),
                                          float(sc["fast"]), float(sc["slow"]))
        return f, mult, dims
    return inv_freq.to(torch.float32), 1.0, dims


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    """Names and shapes of a checkpoint of this config."""
    W, V = int(config["width"]), int(config["vocab"])
    layers = config["layers"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    bg = (config.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = (int(bg["buckets"]) + 1, W)
    side = config.get("token_side")
    if side:
        out["side.embed"] = (V, len(layers) * int(side["dim"]))
    for i, L in enumerate(layers):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (W,)
        out[p + "dwa"] = (i + 2,)
        if side:
            sd = int(side["dim"])
            out.update({p + "side.gate": (sd, W), p + "side.proj": (W, sd), p + "side.norm": (W,)})
        if L["type"] == "attention":
            H, G, dim, vd = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
            out.update({p + "mix.q": (H * 2 * dim, W), p + "mix.q.norm": (dim,), p + "mix.g": (H, W),
                        p + "mix.o": (W, H * vd)})
            out.update({p + f"mix.{k}": (dim,) for k in ("lq1", "lk1", "lq2", "lk2")})
            if m.get("kv_from") is None:
                out.update({p + "mix.k": (G * 2 * dim, W), p + "mix.v": (G * vd, W), p + "mix.k.norm": (dim,)})
        elif L["type"] == "mingru":
            n = int(m["width"])
            out.update({p + "mix.z": (n, W), p + "mix.z.b": (n,), p + "mix.x": (n, W), p + "mix.x.b": (n,),
                        p + "mix.g": (n, W), p + "mix.o": (W, n)})
        else:
            raise ValueError(f"unknown mixer type {L['type']!r}")
        mlp = L.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] != "dense":
            raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
        ff = int(mlp["ff"])
        out.update({p + "norm2": (W,), p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    return out


def random_tensors(config: dict, seed: int = 0, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights of the architecture (bench and tests): projections N(0, 1/in), small vectors."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if leaf == "dwa":
            t = torch.full(shape, 1.0 / shape[0]) + 0.1 * torch.randn(shape, generator=g)
            t[-1] += 0.5
        elif leaf in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram", "side.embed"):
            t = torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


class _Layer:
    kind: str = ""
    mixer = None
    norm1: PostNormResidual
    ff = None
    norm2: Optional[PostNormResidual] = None
    side: Optional[TokenSideInput] = None
    dwa: Optional[torch.Tensor] = None
    cache: Optional[KVCache] = None       # this layer's own, or the one of the layer it takes keys and values from
    kv_from: Optional[int] = None


@register_model("Pokadra")
class PokadraDecoder:
    needs_state_slots = True
    needs_prev_token = True
    CSRC = ("postnorm.cu", "mingru.cu", "diff_attn.cu")

    def __init__(self, config: dict, dtype: torch.dtype, device, max_seqs: int = 4):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Pokadra runs in bfloat16 or float32")
        _lib.ensure(self.CSRC)
        self.config, self.dtype, self.device, self.max_seqs = config, dtype, torch.device(device), max_seqs
        self.width, self.n_vocab = int(config["width"]), int(config["vocab"])
        self.eps = float(config["norm"]["eps"])
        self.groups = int(config["norm"].get("groups", 1))
        self.mult = float(config.get("residual_mult", 1.0))
        emb = config.get("embedding") or {}
        self.embed_scale = float(emb.get("scale", 1.0))
        self.bigram_cfg = emb.get("bigram")
        self.layers: List[_Layer] = []
        self.embed = self.bigram = self.final_norm = self.head = None
        self.use_history = False

    @classmethod
    def from_config(cls, config: dict, dtype, device, max_seqs: int = 4) -> "PokadraDecoder":
        return cls(config, dtype, device, max_seqs)

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0) -> None:
        self.load_weights(random_tensors(self.config, seed))

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        dev, dt, eps = self.device, self.dtype, self.eps
        missing = [n for n in tensor_shapes(self.config) if n not in tensors and not n.endswith(".dwa")]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        w = lambda name: tensors[name].to(dev).to(dt)
        f32 = lambda name: tensors[name].to(dev).to(torch.float32).contiguous()
        self.embed = w("embed").contiguous()
        self.bigram = w("bigram").contiguous() if self.bigram_cfg else None
        self.final_norm = f32("final.norm")
        self.head = Linear(w("head"))
        side_cfg = self.config.get("token_side")
        side_table = w("side.embed").contiguous() if side_cfg else None
        self.layers = []
        for i, L in enumerate(self.config["layers"]):
            p, m = f"l{i}.", L["mixer"]
            lay = _Layer()
            lay.kind = L["type"]
            mw = {k[len(p) + 4:]: w(k) for k in tensors if k.startswith(p + "mix.")}
            if L["type"] == "attention":
                inv_freq, mult, dims = rotary_table(m.get("rot"))
                mask = m.get("mask") or {}
                lay.kv_from = None if m.get("kv_from") is None else int(m["kv_from"])
                if lay.kv_from is not None:
                    if not (0 <= lay.kv_from < i and self.config["layers"][lay.kv_from]["type"] == "attention"):
                        raise ValueError(f"layer {i}: kv_from must name an earlier attention layer")
                    mw = {k: v for k, v in mw.items() if k not in ("k", "v", "k.norm")}
                lay.mixer = DiffAttention(mw, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]),
                                          float(m["scale"]), int(mask.get("size", 0)), int(mask.get("keep_first", 0)),
                                          float(m["diff"]), inv_freq, mult, dims, eps, dt, dev)
            elif L["type"] == "mingru":
                lay.mixer = MinGRUMixer(mw, self.max_seqs, dt, dev)
            else:
                raise ValueError(f"unknown mixer type {L['type']!r}")
            lay.norm1 = PostNormResidual(f32(p + "norm1"), self.groups, self.mult, eps)
            mlp = L.get("mlp")
            if mlp is not None:
                if mlp["kind"] != "dense":
                    raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
                f = p + "mlp."
                lay.ff = ClampedGLU(w(f + "gate"), w(f + "up"), w(f + "down"), float(mlp["limit"]), GLU_SLOPE)
                lay.norm2 = PostNormResidual(f32(p + "norm2"), self.groups, self.mult, eps)
            if side_cfg:
                sd = int(side_cfg["dim"])
                lay.side = TokenSideInput(side_table, i * sd, w(p + "side.gate"), w(p + "side.proj"),
                                          PostNormResidual(f32(p + "side.norm"), 1, self.mult, eps))
            if p + "dwa" in tensors:
                lay.dwa = f32(p + "dwa")
            self.layers.append(lay)
        self.use_history = any(lay.dwa is not None for lay in self.layers)

    # ------------------------------------------------------------------ cache
    def alloc_cache(self, n_blocks: int, block_size: int) -> None:
        for lay, L in zip(self.layers, self.config["layers"]):
            if L["type"] == "attention" and lay.kv_from is None:
                m = L["mixer"]
                lay.cache = KVCache(n_blocks, block_size, int(m["kv_heads"]), 2 * int(m["dim"]), self.dtype,
                                    self.device, value_dim=int(m["vdim"]))
        for lay in self.layers:
            if lay.kv_from is not None:
                lay.cache = self.layers[lay.kv_from].cache

    # ------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, params: InputParameters,
                last_token_idxes: Optional[torch.Tensor] = None, layer_out: Optional[list] = None) -> torch.Tensor:
        """One step over the packed rows of all sequences; logits [rows or len(last_token_idxes), vocab].
        layer_out, if given, receives what every layer hands on (fp32, after the depth average)."""
        T, W, n_layers = tokens.numel(), self.width, len(self.layers)
        bg = self.bigram_cfg or {}
        hist = torch.empty((n_layers + 1, T, W), dtype=torch.float32, device=self.device) if self.use_history else None
        x, h = kernels.bigram_embed(self.embed, self.bigram, tokens, params.prev_tokens, int(bg.get("buckets", 0)),
                                    int(bg.get("mul_prev", 0)), int(bg.get("mul_cur", 0)), self.embed_scale,
                                    x_out=hist[0] if hist is not None else None)
        h = x if h is None else h
        work = torch.empty((T, W), dtype=torch.float32, device=self.device) if hist is not None else x
        for i, lay in enumerate(self.layers):
            subs = [("mix", lay.norm1)]
            if lay.ff is not None:
                subs.append(("ff", lay.norm2))
            if lay.side is not None:
                subs.append(("side", None))
            for n, (kind, norm) in enumerate(subs):
                kw = {"x_out": work}
                if n == len(subs) - 1 and hist is not None:
                    if lay.dwa is not None:
                        kw = {"x_out": work, "hist": hist, "n_hist": i + 2, "coef": lay.dwa}
                    else:       # no average after this layer: its result goes on and into the history
                        kw = {"x_out": hist[i + 1]}
                if kind == "side":
                    x, h = lay.side(x, h, tokens, **kw)
                    continue
                if kind == "mix":
                    y = (lay.mixer(h, positions, lay.cache, params) if lay.kind == "attention"
                         else lay.mixer(h, positions, params))
                else:
                    y = lay.ff(h)
                x, h = norm(x, y, **kw)
            if layer_out is not None:
                layer_out.append(x.clone())
        if last_token_idxes is not None:
            x = x.index_select(0, last_token_idxes.to(torch.int64))
        return self.head(kernels.group_rms_norm(x, self.final_norm, self.groups, self.eps, self.dtype))

    __call__ = forward
