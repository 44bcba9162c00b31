"""Small Kigalix configurations and weights for the tests (not the product's generator: shapes are derived
here from the config, so the product's own shape table is checked against this one)."""
import math

import torch


def latent(heads, dim, rot_dim, vdim, rank, yarn=False, gate=False, base=10000.0, dims=None, scale=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if yarn:
        rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}
    return {"type": "latent_attention_2" if gate or yarn else "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "rot": rot,
                      "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}}


def delta(heads, dim):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, width=64, vocab=97, streams=2, eps=1e-5):
    """layers: list of (mixer entry, mlp entry or None)."""
    return {"architecture": "Kigalix", "width": width, "vocab": vocab, "streams": streams, "norm": {"eps": eps},
            "layers": [dict(m, mlp=f) for m, f in layers]}


def shapes(cfg, decay_rank=8):
    W, V, S = cfg["width"], cfg["vocab"], cfg["streams"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for q in ((1, 2) if L["mlp"] is not None else (1,)):
            out.update({f"{p}norm{q}": (W,), f"{p}rg{q}": (W, W), f"{p}rg{q}.b": (W,), f"{p}hc{q}.in": (S,),
                        f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
        out[p + "shift"] = (W,)
        if L["type"].startswith("latent"):
            H, d, r, v, k = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H * (d + r), W), p + "mix.dkv": (k + r, W), p + "mix.dkv.norm": (k,),
                        p + "mix.uk": (H * d, k), p + "mix.uv": (H * v, k), p + "mix.o": (W, H * v)})
            if L["type"].endswith("_2"):
                out[p + "mix.g"] = (H * v, W)
        else:
            n = m["heads"] * m["dim"]
            for leaf in "rkvga":
                out[p + "mix." + leaf] = (n, W)
            out.update({p + "mix.a.b": (n,), p + "mix.w1": (decay_rank, W), p + "mix.w2": (n, decay_rank),
                        p + "mix.w0": (n,), p + "mix.norm": (n,), p + "mix.o": (W, n)})
        f = L["mlp"]
        if f is None:
            continue
        if f["kind"] == "dense":
            out.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        else:
            out[p + "mlp.router"] = (f["router"]["experts"], W)
            for e in range(f["router"]["experts"]):
                out.update({p + f"mlp.e{e}.gate": (f["expert"]["ff"], W), p + f"mlp.e{e}.up": (f["expert"]["ff"], W),
                            p + f"mlp.e{e}.down": (W, f["expert"]["ff"])})
    return out


def weights(cfg, seed=0):
    """bf16 tensors: projections N(0, 1/in) (queries and keys a little larger so that attention is peaked),
    stream coefficients near the plain residual, everything else small."""
    g = torch.Generator().manual_seed(seed)
    S = cfg["streams"]
    out = {}
    for name, shp in shapes(cfg).items():
        leaf = name.split(".")[-1]
        if ".hc" in name and leaf == "mix":
            t = torch.eye(S) + 0.2 * torch.randn(shp, generator=g)
        elif ".hc" in name and leaf == "in":
            t = torch.full(shp, 1.0 / S) + 0.2 * torch.randn(shp, generator=g)
        elif ".hc" in name and leaf == "out":
            t = 1.0 + 0.2 * torch.randn(shp, generator=g)
        elif leaf == "shift":
            t = torch.rand(shp, generator=g)
        elif name == "embed":
            t = torch.randn(shp, generator=g)
        elif len(shp) == 1:
            t = 0.3 * torch.randn(shp, generator=g)
        elif leaf in ("q", "dkv", "router"):
            t = 2.0 * torch.randn(shp, generator=g) / math.sqrt(shp[-1])
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


# the configurations the model-level tests run: every mixer and feed-forward kind, head counts and sizes that
# are not powers of two, 1 to 3 streams, top 1 and 2, a layer without feed-forward, rotary dims below rot_dim
CONFIGS = {
    "mix": config([(latent(3, 16, 8, 12, 24, yarn=True, gate=True), dense(80)),
                   (delta(2, 24), moe(4, 2, 40)),
                   (latent(5, 8, 4, 8, 40), moe(6, 1, 24)),
                   (delta(3, 16), None)], width=64, vocab=97, streams=2),
    "one_stream": config([(delta(1, 32), dense(48)), (latent(2, 32, 16, 32, 64, dims=8), moe(3, 3, 32))],
                         width=48, vocab=61, streams=1),
    "three_streams": config([(latent(4, 24, 8, 16, 72, gate=True), moe(5, 2, 56)), (delta(4, 40), dense(96))],
                            width=96, vocab=130, streams=3, eps=1e-6),
}
