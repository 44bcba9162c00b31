"""GPU: the Kigalix decoder through the serving engine against the plain CPU restatement (oracle/kigalix.py,
float64): every mechanism alone, whole prompts, token-by-token decoding, portions, mixed batches, reuse of
blocks and state slots, far keys and block borders, generation through the scheduler."""
import math

import numpy as np
import pytest
import torch

from oracle import kigalix as ok
from tests import kigalix_case as kc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None
TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]


def build(cfg, dtype, seed=0, max_seqs=4):
    from scalellm_b200 import registry
    w = kc.weights(cfg, seed)
    model = registry.create_model(cfg, dtype, DEV, max_seqs=max_seqs)
    model.load_weights({k: v.to(DEV) for k, v in w.items()})
    return model, ok.Kigalix(cfg, w)


def engine_for(model, max_tokens=512, block_size=4, max_seqs=4, use_graphs=False):
    from scalellm_b200.engine import Engine
    return Engine(model, max_tokens, block_size=block_size, max_seqs=max_seqs, use_graphs=use_graphs)


def oracle_logits(oracle, tokens):
    return oracle.forward(tokens, oracle.new_state())


def run_schedule(eng, tokens, cuts, rid="r"):
    """Feed `tokens` in portions of the given sizes (the rest one by one); logits of every position."""
    from scalellm_b200.engine import StepEntry
    out, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(tokens) - at)
        out.append(eng.step([StepEntry(rid, tokens[at:at + n], list(range(n)))]).float().cpu())
        at += n
    eng.finish(rid)
    return torch.cat(out, 0)


def toks(n, vocab, seed):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, size=n)]


# ------------------------------------------------------------------ mechanisms alone
def _params(n_tokens_per_seq, cached, block_size=4, n_blocks=256, slots=None):
    from scalellm_b200.decode_step import BlockPool, StepBuffers, build_step_batch
    pool = BlockPool(n_blocks, block_size, seed=3)
    seqs = []
    for n, c in zip(n_tokens_per_seq, cached):
        s = pool.open_sequence()
        pool.reserve(s, n + c)
        seqs.append(s)
    hb = build_step_batch(pool, seqs, [[0] * n for n in n_tokens_per_seq], list(cached),
                          slots if slots is not None else list(range(len(seqs))))
    bufs = StepBuffers(DEV, sum(n_tokens_per_seq) + 8, len(seqs) + 1, n_blocks + 8)
    return bufs.upload(hb), hb


@pytest.mark.parametrize("S,W", [(1, 48), (2, 64), (3, 200)])
def test_stream_collapse_norm_and_gated_update(S, W):
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(S * 100 + W)
    X = torch.randn(7, S, W, generator=g)
    a, wn = torch.randn(S, generator=g), 0.3 * torch.randn(W, generator=g)
    n = kernels.hc_norm(X.to(DEV), a.to(DEV), wn.to(DEV), 1e-5, 1.0, torch.float32)
    u = (X.double() * a.double()[None, :, None]).sum(1)
    ref = ok.offset_norm(u, wn.double(), 1e-5)
    assert float((n.cpu().double() - ref).abs().max()) < 1e-5
    y, gl, gb = torch.randn(7, W, generator=g), torch.randn(7, W, generator=g), torch.randn(W, generator=g)
    M, b = torch.randn(S, S, generator=g), torch.randn(S, generator=g)
    Xd = X.to(DEV).clone()
    kernels.gated_hc_update(Xd, y.to(DEV), gl.to(DEV), gb.to(DEV), M.to(DEV), b.to(DEV))
    yy = y.double() * torch.sigmoid(gl.double() + gb.double())
    ref = torch.einsum("st,rsw->rtw", M.double(), X.double()) + b.double()[None, :, None] * yy[:, None, :]
    assert float((Xd.cpu().double() - ref).abs().max()) < 1e-5


def test_token_shift_state_across_portions_and_slots():
    """Two sequences in two steps; the second step's first rows must read what the first step left in
    each sequence's own slot, and a sequence that starts at position 0 must not read its slot at all."""
    from scalellm_b200.layers import TokenShift
    W = 40
    g = torch.Generator().manual_seed(1)
    mu = torch.rand(W, generator=g)
    ts = TokenShift(mu.to(DEV), 4, torch.float32, DEV)
    ts.state.fill_(123.0)                                    # stale content of reused slots
    n_a, n_b = torch.randn(9, W, generator=g), torch.randn(5, W, generator=g)
    ref_a, _ = ok.token_shift(n_a.double(), torch.zeros(W, dtype=torch.float64), mu.double())
    ref_b, _ = ok.token_shift(n_b.double(), torch.zeros(W, dtype=torch.float64), mu.double())
    (tk, pos, prm), _ = _params([6, 2], [0, 0], slots=[2, 0])
    out1 = ts(torch.cat([n_a[:6], n_b[:2]]).to(DEV), pos, prm).cpu().double()
    (tk, pos, prm), _ = _params([3, 3], [6, 2], slots=[2, 0])
    out2 = ts(torch.cat([n_a[6:], n_b[2:]]).to(DEV), pos, prm).cpu().double()
    got_a, got_b = torch.cat([out1[:6], out2[:3]]), torch.cat([out1[6:], out2[3:]])
    assert float((got_a - ref_a).abs().max()) < 1e-6 and float((got_b - ref_b).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dim,rd,vd,rank,dims,yarn", [(3, 16, 8, 12, 24, 8, True), (5, 8, 4, 8, 40, 4, False),
                                                         (2, 32, 16, 32, 64, 8, False), (9, 24, 12, 20, 100, 12, True)])
def test_latent_attention_far_key_and_block_borders(dtype, H, dim, rd, vd, rank, dims, yarn):
    """One long sequence in two portions (cut inside a block).  The input rows are made so that the last
    query points at one far key: rows 5 and T-1 share a large common direction.  A key that is skipped, read
    from the wrong block or rotated with the wrong position changes the output visibly."""
    from scalellm_b200.layers import LatentAttention, LatentKVCache
    from scalellm_b200.kigalix import rotary_table
    W, T, cut, bs = 64, 333, 202, 8
    mcfg = kc.latent(H, dim, rd, vd, rank, yarn=yarn, gate=yarn, dims=dims)["mixer"]
    g = torch.Generator().manual_seed(H * 7 + rank)
    names = {"q": (H * (dim + rd), W), "dkv": (rank + rd, W), "dkv.norm": (rank,), "uk": (H * dim, rank),
             "uv": (H * vd, rank), "o": (W, H * vd)}
    if yarn:
        names["g"] = (H * vd, W)
    w = {k: (torch.randn(s, generator=g) / math.sqrt(s[-1]) if len(s) == 2 else 1 + 0.2 * torch.randn(s, generator=g)
             ).to(torch.bfloat16) for k, s in names.items()}
    h0 = torch.randn(T, W, generator=g)
    spike = torch.randn(W, generator=g)
    wd = {k: v.double() for k, v in w.items()}
    best = None
    for sign in (1.0, -1.0):            # random maps: which sign makes the last query point AT row 5 is found by trying
        h = h0.clone()
        h[5] += 6 * spike
        h[T - 1] += sign * 6 * spike
        h = h.to(torch.bfloat16)
        ref = ok.latent_attention(h.double(), torch.arange(T), wd, mcfg, 1e-5, {})
        h2 = h.clone()
        h2[5] = 0
        ref2 = ok.latent_attention(h2.double(), torch.arange(T), wd, mcfg, 1e-5, {})
        effect = float((ref2[-1] - ref[-1]).abs().max() / ref.abs().max())
        if best is None or effect > best[0]:
            best = (effect, h, ref)
    effect, h, ref = best
    assert effect > 0.03                # the far key carries a visible share of the last row's output
    inv_freq, mult = rotary_table(mcfg["rot"])
    layer = LatentAttention({k: v.to(DEV).to(dtype) for k, v in w.items()}, H, dim, rd, vd, rank, mcfg["scale"],
                            inv_freq, mult, dims, 1e-5, dtype, DEV)
    cache = LatentKVCache(64, bs, rank, rd, dtype, DEV)
    (tk, pos, prm), _ = _params([cut], [0], block_size=bs, n_blocks=64)
    o1 = layer(h[:cut].to(DEV).to(dtype), pos, cache, prm)
    from scalellm_b200.decode_step import BlockPool, StepBuffers, build_step_batch
    pool = BlockPool(64, bs, seed=3)                         # same seed: same blocks as the first portion
    s = pool.open_sequence()
    pool.reserve(s, T)
    hb = build_step_batch(pool, [s], [[0] * (T - cut)], [cut], [0])
    tk, pos, prm = StepBuffers(DEV, T, 2, 80).upload(hb)
    o2 = layer(h[cut:].to(DEV).to(dtype), pos, cache, prm)
    got = torch.cat([o1, o2]).float().cpu().double()
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < (3e-5 if dtype == torch.float32 else 3e-2), err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d", [(2, 24), (1, 32), (3, 48), (2, 64), (1, 100)])
def test_delta_rule_portions_and_state(dtype, H, d):
    from scalellm_b200.layers import DeltaRuleMixer
    W, T = 48, 70
    g = torch.Generator().manual_seed(H * 31 + d)
    n = H * d
    shp = {"r": (n, W), "k": (n, W), "v": (n, W), "g": (n, W), "a": (n, W), "a.b": (n,), "w1": (8, W), "w2": (n, 8),
           "w0": (n,), "norm": (n,), "o": (W, n)}
    w = {k: (torch.randn(s, generator=g) / math.sqrt(s[-1]) if len(s) == 2 else 0.5 * torch.randn(s, generator=g)
             ).to(torch.bfloat16) for k, s in shp.items()}
    h = torch.randn(T, W, generator=g).to(torch.bfloat16)
    ref = ok.general_delta(h.double(), {k: v.double() for k, v in w.items()}, {"heads": H, "dim": d}, 1e-5, {})
    from scalellm_b200.kigalix import DELTA_DECAY_SCALE, DELTA_KEY_EPS
    layer = DeltaRuleMixer({k: v.to(DEV).to(dtype) for k, v in w.items()}, H, d, DELTA_DECAY_SCALE, DELTA_KEY_EPS,
                           1e-5, 3, dtype, DEV)
    layer.state.fill_(7.0)                                   # a reused slot is not cleared by anyone
    outs, at = [], 0
    for nq in (33, 2, 1, 1, 30, 3):
        (tk, pos, prm), _ = _params([nq], [at], slots=[1])
        outs.append(layer(h[at:at + nq].to(DEV).to(dtype), pos, prm))
        at += nq
    got = torch.cat(outs).float().cpu().double()
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < (3e-5 if dtype == torch.float32 else 3e-2), err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,ff,rows", [(4, 1, 40, 50), (6, 2, 24, 200), (3, 3, 70, 9), (8, 2, 96, 1)])
def test_experts_route_on_input_scaled_rows(dtype, E, top, ff, rows):
    from scalellm_b200.layers import SparseMoE
    W = 64
    g = torch.Generator().manual_seed(E * 13 + top)
    router = (3 * torch.randn(E, W, generator=g) / math.sqrt(W)).to(torch.bfloat16)
    gate, up = (torch.randn(E, ff, W, generator=g) / 8).to(torch.bfloat16), (torch.randn(E, ff, W, generator=g) / 8).to(torch.bfloat16)
    down = (torch.randn(E, W, ff, generator=g) / math.sqrt(ff)).to(torch.bfloat16)
    h = torch.randn(rows, W, generator=g).to(torch.bfloat16)
    w = {"router": router.double()}
    for e in range(E):
        w.update({f"e{e}.gate": gate[e].double(), f"e{e}.up": up[e].double(), f"e{e}.down": down[e].double()})
    ref = ok.moe_ff(h.double(), w, {"router": {"experts": E, "top": top}})
    layer = SparseMoE(router.to(DEV), gate.to(DEV).to(dtype), up.to(DEV).to(dtype), down.to(DEV).to(dtype), top, "silu")
    got = layer(h.to(DEV).to(dtype)).float().cpu().double()
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < (3e-5 if dtype == torch.float32 else 3e-2), err


def test_dense_feed_forward_uses_the_tanh_gelu():
    from scalellm_b200.layers import GatedMLP
    g = torch.Generator().manual_seed(4)
    W, ff = 48, 112
    gate, up, down = (torch.randn(s, generator=g) / 6 for s in ((ff, W), (ff, W), (W, ff)))
    h = 2 * torch.randn(19, W, generator=g)
    ref = ok.dense_ff(h.double(), {"gate": gate.double(), "up": up.double(), "down": down.double()})
    got = GatedMLP(gate.to(DEV), up.to(DEV), down.to(DEV), "gelu_tanh")(h.to(DEV)).cpu().double()
    assert float((got - ref).abs().max() / ref.abs().max()) < 2e-5


# ------------------------------------------------------------------ the model through the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(kc.CONFIGS))
def test_whole_prompt_decode_and_portions_match_the_oracle(name, dtype):
    cfg = kc.CONFIGS[name]
    model, oracle = build(cfg, dtype, seed=1)
    tokens = toks(75, cfg["vocab"], 11)
    ref = oracle_logits(oracle, tokens)
    eng = engine_for(model, block_size=4)
    for cuts in ([75], [40], [2, 2, 3, 17, 1, 30, 2], [1, 1, 1, 9, 8, 7, 33, 2, 2]):   # the rest one token at a time
        got = run_schedule(eng, tokens, cuts)
        assert kc.logits_error(got, ref) < TOL[dtype], (name, cuts)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_batches_equal_each_request_alone_and_reuse_blocks_and_slots(dtype):
    """Three unequal requests interleaved (portions beside decoded tokens) in an engine with a pool too small
    for all of them at once and two state slots: the third is admitted into what the first gave back."""
    from scalellm_b200.engine import StepEntry
    cfg = kc.CONFIGS["mix"]
    model, oracle = build(cfg, dtype, seed=2, max_seqs=2)
    reqs = {"a": toks(41, cfg["vocab"], 1), "b": toks(23, cfg["vocab"], 2), "c": toks(37, cfg["vocab"], 3)}
    ref = {k: oracle_logits(oracle, v) for k, v in reqs.items()}
    eng = engine_for(model, max_tokens=72, block_size=4, max_seqs=2)
    got = {k: [] for k in reqs}
    at = {k: 0 for k in reqs}

    def step(plan):
        entries = [StepEntry(k, reqs[k][at[k]:at[k] + n], list(range(n))) for k, n in plan]
        out = eng.step(entries).float().cpu()
        r = 0
        for k, n in plan:
            got[k].append(out[r:r + n])
            r += n
            at[k] += n
            if at[k] == len(reqs[k]):
                eng.finish(k)
    step([("a", 30)])
    step([("a", 1), ("b", 7)])
    step([("b", 2), ("a", 1)])
    for _ in range(9):
        step([("a", 1), ("b", 1)])                       # a ends here
    step([("c", 20), ("b", 1)])                          # c takes a's blocks and slot
    step([("b", 4), ("c", 2)])
    while at["b"] < len(reqs["b"]) or at["c"] < len(reqs["c"]):
        step([(k, 1) for k in ("c", "b") if at[k] < len(reqs[k])])
    assert eng.pool.n_free_blocks() == 18 and len(eng.slots.free) == 2
    for k in reqs:
        assert kc.logits_error(torch.cat(got[k]), ref[k]) < TOL[dtype], k
    alone = engine_for(build(cfg, dtype, seed=2)[0], block_size=4)
    for k in reqs:
        assert kc.logits_error(torch.cat(got[k]), run_schedule(alone, reqs[k], [len(reqs[k])])) < TOL[dtype] / 2, k


def test_long_decoding_over_many_blocks():
    cfg = kc.CONFIGS["three_streams"]
    model, oracle = build(cfg, torch.float32, seed=5)
    tokens = toks(140, cfg["vocab"], 9)
    got = run_schedule(engine_for(model, block_size=2), tokens, [3])      # 137 single-token steps
    assert kc.logits_error(got, oracle_logits(oracle, tokens)) < TOL[torch.float32]


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_by_graph_replay(dtype):
    """Single-token steps replay a captured graph from the third step on; two sequences decode side by side,
    and a third batch size (one sequence left) gets a graph of its own."""
    from scalellm_b200.engine import StepEntry
    cfg = kc.CONFIGS["mix"]
    model, oracle = build(cfg, dtype, seed=8)
    a, b = toks(48, cfg["vocab"], 21), toks(30, cfg["vocab"], 22)
    ref_a, ref_b = oracle_logits(oracle, a), oracle_logits(oracle, b)
    eng = engine_for(model, block_size=4, use_graphs=True)
    out = eng.step([StepEntry("a", a[:20], list(range(20))), StepEntry("b", b[:9], list(range(9)))]).float().cpu()
    got_a, got_b = [out[:20]], [out[20:]]
    for i in range(21):                                   # b ends first
        out = eng.step([StepEntry("b", [b[9 + i]], [0]), StepEntry("a", [a[20 + i]], [0])]).float().cpu()
        got_b.append(out[:1])
        got_a.append(out[1:])
    eng.finish("b")
    for i in range(41, 48):
        got_a.append(eng.step([StepEntry("a", [a[i]], [0])]).float().cpu())
    assert len(eng._graphs) == 2
    assert kc.logits_error(torch.cat(got_a), ref_a) < TOL[dtype]
    assert kc.logits_error(torch.cat(got_b), ref_b) < TOL[dtype]


def test_the_first_tokens_of_a_sequence():
    """Positions 0 and 1 alone, in a slot and blocks that an earlier request left dirty."""
    cfg = kc.CONFIGS["mix"]
    model, oracle = build(cfg, torch.float32, seed=6, max_seqs=1)
    eng = engine_for(model, max_tokens=32, block_size=4, max_seqs=1)
    run_schedule(eng, toks(30, cfg["vocab"], 1), [30], rid="old")
    tokens = toks(6, cfg["vocab"], 2)
    got = run_schedule(eng, tokens, [1, 1, 2, 2], rid="new")
    assert kc.logits_error(got, oracle_logits(oracle, tokens)) < TOL[torch.float32]


def test_greedy_generation_through_the_scheduler():
    from scalellm_b200.engine import SamplingParams
    cfg = kc.CONFIGS["mix"]
    model, oracle = build(cfg, torch.float32, seed=7)
    prompts = [toks(n, cfg["vocab"], n) for n in (19, 5, 33, 12, 7)]      # more requests than sequence places
    eng = engine_for(model, max_tokens=160, block_size=4, max_seqs=3)
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=n) for n in (6, 9, 4, 7, 5)], max_step_tokens=16)
    for p, o in zip(prompts, outs):
        seq, st = list(p), oracle.new_state()
        lg = oracle.forward(seq, st)[-1]
        for t in o:
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > 1e-3 * float(lg.abs().max()):   # a near tie may fall either way
                assert t == int(lg.argmax())
            lg = oracle.forward([t], st)[-1]
    assert eng.pool.n_free_blocks() == 40 and not eng.seqs


def test_sampled_generation_is_seeded_and_top_k_one_is_greedy():
    from scalellm_b200.engine import SamplingParams
    cfg = kc.CONFIGS["one_stream"]
    model, _ = build(cfg, torch.bfloat16, seed=9)
    prompts = [toks(9, cfg["vocab"], 1), toks(4, cfg["vocab"], 2)]
    gen = lambda sp: engine_for(model, max_tokens=128, block_size=4).generate(prompts, sp)
    greedy = gen([SamplingParams(max_new_tokens=5)] * 2)
    assert gen([SamplingParams(5, temperature=0.8, top_k=1, seed=3)] * 2) == greedy
    a = gen([SamplingParams(5, temperature=1.5, top_k=20, top_p=0.95, seed=3), SamplingParams(5, temperature=1.5, seed=4)])
    b = gen([SamplingParams(5, temperature=1.5, top_k=20, top_p=0.95, seed=3), SamplingParams(5, temperature=1.5, seed=4)])
    assert a == b and all(0 <= t < cfg["vocab"] for o in a for t in o)


def test_llama_runs_through_the_same_engine():
    """The Llama decoder behind the registry and the engine: a prompt in portions plus decoded tokens gives
    the logits of the whole prompt in one step (same kernels, other cuts), and blocks are reused."""
    from scalellm_b200 import registry
    cfg = {"architectures": ["LlamaForCausalLM"], "hidden_size": 256, "num_hidden_layers": 2,
           "num_attention_heads": 2, "num_key_value_heads": 1, "intermediate_size": 512, "vocab_size": 512,
           "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 512, "rope_scaling": None}
    model = registry.create_model(cfg, torch.bfloat16, DEV, max_seqs=2)
    model.init_random(3)
    tokens = toks(40, 512, 5)
    eng = engine_for(model, max_tokens=64, block_size=8, max_seqs=2)
    whole = run_schedule(eng, tokens, [40])
    parts = run_schedule(eng, tokens, [9, 17, 2])
    assert eng.pool.n_free_blocks() == 8 and eng.slots is None
    assert kc.logits_error(parts, whole) < 3e-2


def test_unknown_architecture_and_layer_type_are_refused():
    from scalellm_b200 import registry
    with pytest.raises(ValueError):
        registry.model_class({"architecture": "NoSuchModel"})
    bad = kc.config([({"type": "conv_mixer", "mixer": {}}, None)])
    with pytest.raises((ValueError, KeyError)):
        registry.create_model(bad, torch.float32, DEV).load_weights({})
