"""Small Pokadra configurations and weights for the tests (not the product's generator: shapes are derived
here from the config, so the product's own shape table is checked against this one)."""
import math

import torch


def attn(heads, kv_heads, dim, vdim, window=None, keep_first=0, rot_dims=None, yarn=False, diff=0.5, kv_from=None,
         base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if yarn:
            m["rot"]["scaling"] = {"factor": 8.0, "original": 32, "fast": 8.0, "slow": 2.0}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def dense(ff, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(layers, width=64, vocab=97, groups=2, eps=1e-5, mult=0.5, scale=2.0, bigram=(53, 31, 5), side=8):
    """layers: list of (mixer entry, mlp entry or None); bigram: (buckets, mul_prev, mul_cur) or None."""
    cfg = {"architecture": "Pokadra", "width": width, "vocab": vocab, "norm": {"eps": eps, "groups": groups},
           "residual_mult": mult, "embedding": {"scale": scale}, "layers": [dict(m, mlp=f) for m, f in layers]}
    if bigram:
        cfg["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def shapes(cfg):
    W, V, n = cfg["width"], cfg["vocab"], len(cfg["layers"])
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if "bigram" in cfg["embedding"]:
        out["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    sd = cfg["token_side"]["dim"] if "token_side" in cfg else 0
    if sd:
        out["side.embed"] = (V, n * sd)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"], out[p + "dwa"] = (W,), (i + 2,)
        if sd:
            out.update({p + "side.gate": (sd, W), p + "side.proj": (W, sd), p + "side.norm": (W,)})
        if L["type"] == "attention":
            H, G, d, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (2 * H * d, W), p + "mix.q.norm": (d,), p + "mix.g": (H, W), p + "mix.o": (W, H * v),
                        p + "mix.lq1": (d,), p + "mix.lk1": (d,), p + "mix.lq2": (d,), p + "mix.lk2": (d,)})
            if "kv_from" not in m:
                out.update({p + "mix.k": (2 * G * d, W), p + "mix.v": (G * v, W), p + "mix.k.norm": (d,)})
        else:
            n_ = m["width"]
            out.update({p + "mix.z": (n_, W), p + "mix.z.b": (n_,), p + "mix.x": (n_, W), p + "mix.x.b": (n_,),
                        p + "mix.g": (n_, W), p + "mix.o": (W, n_)})
        f = L["mlp"]
        if f is not None:
            out.update({p + "norm2": (W,), p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W),
                        p + "mlp.down": (W, f["ff"])})
    return out


def weights(cfg, seed=0):
    """bf16 tensors: projections N(0, 1/in) (queries and keys larger so that attention is peaked and the window's
    edge matters), norm weights around one, averaging coefficients that lean on the newest layer."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shp in shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf == "dwa":
            t = 0.3 * torch.randn(shp, generator=g)
            t[-1] += 1.0
        elif leaf in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.3 * torch.randn(shp, generator=g)
        elif name in ("embed", "bigram", "side.embed"):
            t = torch.randn(shp, generator=g)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.2 * torch.randn(shp, generator=g)
        elif len(shp) == 1:
            t = 0.3 * torch.randn(shp, generator=g)
        elif leaf in ("q", "k") and ".mix." in name:
            t = 3.0 * torch.randn(shp, generator=g) / math.sqrt(shp[-1])
        else:
            t = torch.randn(shp, generator=g) / math.sqrt(shp[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def logits_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest per-row error: rms over the vocabulary of the difference (mean removed) over the rms of the
    expected logits."""
    d = got.double().cpu() - want.double().cpu()
    d = d - d.mean(-1, keepdim=True)
    scale = want.double().pow(2).mean().sqrt()
    return float(d.pow(2).mean(-1).sqrt().max() / scale)


# the configurations the model-level tests run: both mixers in several orders, key/value heads shared by 1, 2 and 3
# query heads, widths that are not powers of two, 1 to 3 norm groups, a layer without feed-forward, layers that
# attend over an earlier layer's keys (adjacent and not), windows 5 to 24 with 0 to 4 kept tokens, full rotation,
# partial rotation, none; with and without the pair table and the per-token term; head sizes that fit the
# tensor-core kernel (multiples of 16) and head sizes that do not
CONFIGS = {
    "mix": config([(gru(40), dense(80)),
                   (attn(4, 2, 16, 32, window=9, keep_first=3, rot_dims=8, yarn=True), dense(48, 1.0)),
                   (gru(72), None),
                   (attn(4, 2, 16, 32, window=5, keep_first=0, rot_dims=8, yarn=True, kv_from=1, diff=0.3), dense(64)),
                   (attn(3, 3, 8, 8, window=24, keep_first=4, rot_dims=8), dense(40))],
                  width=64, vocab=97, groups=2),
    "attn_first": config([(attn(6, 2, 12, 20, rot_dims=4, diff=0.8), dense(56, 0.7)),
                          (gru(30), dense(44)),
                          (attn(6, 2, 12, 20, window=7, keep_first=1, rot_dims=4, kv_from=0), None)],
                         width=48, vocab=61, groups=3, eps=1e-6, mult=1.0, scale=1.0, bigram=None, side=4),
    # every product a multiple of 128 wide and deep: decode-sized bf16 steps hand split-K partials to fused consumers
    "wide": config([(gru(256), dense(128, 1.5)), (attn(4, 2, 16, 32, window=11, keep_first=2, rot_dims=16, yarn=True), dense(256)),
                    (gru(128), None), (attn(4, 2, 16, 32, window=6, keep_first=1, rot_dims=16, yarn=True, kv_from=1), dense(128))],
                   width=128, vocab=160, groups=4, mult=0.4, side=8),
    "plain": config([(attn(2, 1, 32, 48, window=13, keep_first=2), dense(96)), (gru(100), dense(72))],
                    width=80, vocab=130, groups=1, mult=0.25, bigram=(17, 3, 1), side=0),
}
