"""GPU: the Pokadra decoder through the serving engine against the plain CPU restatement (oracle/pokadra.py,
float64): every mechanism alone, whole prompts, token-by-token decoding, portions, mixed batches, reuse of
blocks and state slots, keys far away, at block borders and on both sides of the window's and the kept tokens'
edges, generation through the scheduler."""
import math

import numpy as np
import pytest
import torch

from oracle import pokadra as op
from tests import pokadra_case as pc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None
TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]


def build(cfg, dtype, seed=0, max_seqs=4):
    from scalellm_b200 import registry
    w = pc.weights(cfg, seed)
    model = registry.create_model(cfg, dtype, DEV, max_seqs=max_seqs)
    model.load_weights({k: v.to(DEV) for k, v in w.items()})
    return model, op.Pokadra(cfg, w)


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


def _params(n_tokens_per_seq, cached, block_size=4, n_blocks=256, slots=None, pool_seed=3):
    from scalellm_b200.decode_step import BlockPool, StepBuffers, build_step_batch
    pool = BlockPool(n_blocks, block_size, seed=pool_seed)
    seqs = []
    for n, c in zip(n_tokens_per_seq, cached):
        s = pool.open_sequence()
        pool.reserve(s, n + c)
        seqs.append(s)
    hb = build_step_batch(pool, seqs, [[0] * n for n in n_tokens_per_seq], list(cached),
                          slots if slots is not None else list(range(len(seqs))))
    bufs = StepBuffers(DEV, sum(n_tokens_per_seq) + 8, len(seqs) + 1, n_blocks + 8)
    return bufs.upload(hb), hb


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairs", [True, False])
def test_embedding_with_pair_table(dtype, pairs):
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(1)
    V, W, buckets = 37, 40, 11
    E = torch.randn(V, W, generator=g).to(dtype)
    B = torch.randn(buckets + 1, W, generator=g).to(dtype) if pairs else None
    tokens, prev = [5, 36, 0, 7, 7, 20], [-1, 5, 36, -1, 9, 7]      # two sequence starts, one carried-in token
    x, h = kernels.bigram_embed(E.to(DEV), None if B is None else B.to(DEV), torch.tensor(tokens, dtype=torch.int32, device=DEV),
                                torch.tensor(prev, dtype=torch.int32, device=DEV), buckets, 29, 3, 1.5)
    w = {"embed": E.double(), "bigram": None if B is None else B.double()}
    emb = {"scale": 1.5, "bigram": {"buckets": buckets, "mul_prev": 29, "mul_cur": 3}} if pairs else {"scale": 1.5}
    ref = torch.cat([op.embedding([t], None if p < 0 else p, w, emb) for t, p in zip(tokens, prev)])
    assert float((x.cpu().double() - ref).abs().max()) < 1e-5
    assert (h is None) == (dtype == torch.float32)
    if h is not None:
        assert float((h.cpu().double() - ref).abs().max()) < 0.05


@pytest.mark.parametrize("W,groups", [(48, 1), (64, 4), (200, 5), (96, 96)])
def test_postnorm_residual_and_history(W, groups):
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(W + groups)
    rows, n = 6, 4
    x, y, w = torch.randn(rows, W, generator=g), 3.0 * torch.randn(rows, W, generator=g), torch.randn(W, generator=g)
    y[:, : W // groups] *= 10.0        # one loud group must not change the others
    ref = x.double() + 0.3 * op.group_norm(y.double(), w.double(), groups, 1e-5)
    out, h = kernels.postnorm_residual(x.to(DEV), y.to(DEV), w.to(DEV), groups, 0.3, 1e-5)
    assert h is None and float((out.cpu().double() - ref).abs().max()) < 1e-5
    hist = torch.randn(n + 1, rows, W, generator=g)
    coef = torch.randn(n, generator=g)
    hd = hist.to(DEV)
    out2 = torch.empty(rows, W, device=DEV)
    o, h = kernels.postnorm_residual(x.to(DEV), y.to(torch.bfloat16).to(DEV), w.to(DEV), groups, 0.3, 1e-5, hd, n,
                                     coef.to(DEV), out2)
    refb = x.double() + 0.3 * op.group_norm(y.to(torch.bfloat16).double(), w.double(), groups, 1e-5)
    assert float((hd[n - 1].cpu().double() - refb).abs().max()) < 1e-5            # the stage is stored ...
    assert torch.equal(hd[n].cpu(), hist[n]) and torch.equal(hd[: n - 1].cpu(), hist[: n - 1])   # ... and only it
    avg = sum(coef[j].double() * (refb if j == n - 1 else hist[j].double()) for j in range(n))
    assert float((o.cpu().double() - avg).abs().max()) < 1e-5
    assert h.dtype == torch.bfloat16 and float((h.cpu().double() - avg).abs().max()) < 0.05
    nrm = kernels.group_rms_norm(x.to(DEV), w.to(DEV), groups, 1e-5, torch.float32)
    assert float((nrm.cpu().double() - op.group_norm(x.double(), w.double(), groups, 1e-5)).abs().max()) < 1e-5


def test_clamped_glu_and_token_gate():
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(2)
    gu = 3.0 * torch.randn(9, 2 * 52, generator=g)
    out = kernels.glu_clamped(gu.to(DEV), 1.25, 1.702)
    gg, uu = gu[:, :52].double().clamp(max=1.25), gu[:, 52:].double().clamp(-1.25, 1.25)
    assert float((out.cpu().double() - gg * torch.sigmoid(1.702 * gg) * (uu + 1)).abs().max()) < 1e-5
    for n in (56, 52, 8):       # 16-bit rows of whole 16-byte pieces take the wide kernel, others the plain one
        gb = (3.0 * torch.randn(11, 2 * n, generator=g)).to(torch.bfloat16)
        ob = kernels.glu_clamped(gb.to(DEV), 1.25, 1.702)
        gg, uu = gb[:, :n].double().clamp(max=1.25), gb[:, n:].double().clamp(-1.25, 1.25)
        assert float((ob.cpu().double() - gg * torch.sigmoid(1.702 * gg) * (uu + 1)).abs().max()) < 0.02
    a, table = torch.randn(5, 6, generator=g), torch.randn(13, 30, generator=g)
    tok = [3, 12, 0, 3, 7]
    o = kernels.token_gated_gelu(a.to(DEV), table.to(DEV), 18, torch.tensor(tok, dtype=torch.int32, device=DEV))
    ref = op.gelu_tanh(a.double()) * table.double()[tok, 18:24]
    assert float((o.cpu().double() - ref).abs().max()) < 1e-5


@pytest.mark.parametrize("rows", [1, 7, 128])
def test_consumers_of_split_k_partials(rows):
    """Post-norm and GLU fed by the partials of the product before them against product, then kernel."""
    from scalellm_b200 import kernels
    if not kernels.splitk_consumers_available():
        pytest.skip("the loaded library has no split-K stream kernel")
    g = torch.Generator().manual_seed(rows)
    W, K, n = 256, 384, 128
    a = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    wo = (torch.randn(W, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    x, wn = torch.randn(rows, W, generator=g), torch.randn(W, generator=g)
    hist, coef = torch.randn(3, rows, W, generator=g), torch.randn(2, generator=g)
    y = (a.double() @ wo.double().T).to(torch.bfloat16)
    ref, _ = kernels.postnorm_residual(x.to(DEV), y.to(DEV), wn.to(DEV), 4, 0.3, 1e-5, hist.to(DEV), 2, coef.to(DEV),
                                       torch.empty(rows, W, device=DEV))
    part = kernels.dense_gemm_splitk(a.to(DEV), wo.to(DEV), poison=True)
    hd = hist.to(DEV)
    got, h = kernels.postnorm_residual_splitk(x.to(DEV), part, wn.to(DEV), 4, 0.3, 1e-5, torch.bfloat16, hd, 2,
                                              coef.to(DEV), torch.empty(rows, W, device=DEV))
    assert float((got - ref).abs().max()) < 0.05 and h.dtype == torch.bfloat16      # the sums round to bf16 alike
    assert torch.equal(hd[2].cpu(), hist[2])
    wgu = (torch.randn(2 * n, K, generator=g) / math.sqrt(K) * 3).to(torch.bfloat16)
    gu = (a.double() @ wgu.double().T).to(torch.bfloat16)
    ref = kernels.glu_clamped(gu.to(DEV), 1.5, 1.702)
    got = kernels.glu_clamped_splitk(kernels.dense_gemm_splitk(a.to(DEV), wgu.to(DEV), poison=True), 1.5, 1.702,
                                     torch.bfloat16)
    assert float((got.float() - ref.float()).abs().max()) < 0.06


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,sd,groups", [(64, 8, 1), (200, 12, 4), (48, 1, 3)])
def test_per_token_term_in_one_launch(dtype, W, sd, groups):
    """Gate, projection and post-norm of the per-token term as one kernel, with and without the history."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(W + sd)
    rows, V, layer, n = 5, 23, 2, 3
    x = torch.randn(rows, W, generator=g)
    G_, P_ = (torch.randn(sd, W, generator=g) / math.sqrt(W)).to(dtype), torch.randn(W, sd, generator=g).to(dtype)
    table, wn = torch.randn(V, 4 * sd, generator=g).to(dtype), torch.randn(W, generator=g)
    tok = [3, 22, 0, 3, 9]
    h = x.to(dtype)
    w = {"side.embed": table.double(), "l2.side.gate": G_.double(), "l2.side.proj": P_.double(),
         "l2.side.norm": torch.ones(W, dtype=torch.float64)}
    e = table.double()[tok, layer * sd:(layer + 1) * sd]
    y = (op.gelu_tanh(h.double() @ G_.double().T) * e) @ P_.double().T
    ref = x.double() + 0.4 * op.group_norm(y, wn.double(), groups, 1e-5)
    tol = 1e-4 if dtype == torch.float32 else 0.06
    out, hh = kernels.token_side_postnorm(x.to(DEV), h.to(DEV), G_.to(DEV), P_.t().contiguous().to(DEV), table.to(DEV), layer * sd,
                                          torch.tensor(tok, dtype=torch.int32, device=DEV), wn.to(DEV), groups, 0.4,
                                          1e-5, x_out=torch.empty(rows, W, device=DEV))
    assert float((out.cpu().double() - ref).abs().max()) < tol * (1 + float(ref.abs().max()))
    assert (hh is None) == (dtype == torch.float32)
    hist = torch.randn(n + 1, rows, W, generator=g)
    coef = torch.randn(n, generator=g)
    hd = hist.to(DEV)
    out, _ = kernels.token_side_postnorm(x.to(DEV), h.to(DEV), G_.to(DEV), P_.t().contiguous().to(DEV), table.to(DEV), layer * sd,
                                         torch.tensor(tok, dtype=torch.int32, device=DEV), wn.to(DEV), groups, 0.4,
                                         1e-5, hd, n, coef.to(DEV), torch.empty(rows, W, device=DEV))
    avg = sum(coef[j].double() * (ref if j == n - 1 else hist[j].double()) for j in range(n))
    assert float((out.cpu().double() - avg).abs().max()) < tol * (1 + float(avg.abs().max()))
    assert float((hd[n - 1].cpu().double() - ref).abs().max()) < tol * (1 + float(ref.abs().max()))
    assert torch.equal(hd[n].cpu(), hist[n])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [1, 40, 300])
def test_mingru_in_portions_from_a_dirty_slot(dtype, width):
    """One sequence in portions of 33 / 2 / 1 / 1 / 30 beside a second one that starts later, slots not cleared."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(width)
    n = 67
    proj = (2.0 * torch.randn(n, 3 * width, generator=g)).to(dtype)
    bz, bx = torch.randn(width, generator=g), torch.randn(width, generator=g)
    z = torch.sigmoid(proj[:, :width].double() + bz.double())
    u = proj[:, width:2 * width].double() + bx.double()
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S, ref = torch.zeros(width, dtype=torch.float64), []
    for t in range(n):
        S = (1 - z[t]) * S + z[t] * cand[t]
        gt = proj[t, 2 * width:].double()
        ref.append(S * gt * torch.sigmoid(gt))
    ref = torch.stack(ref)
    tol = (1e-5 if dtype == torch.float32 else 0.01) * (1.0 + float(ref.abs().max()))
    state = torch.full((3, width), 7.0, device=DEV)
    got, at = [], 0
    for k, size in enumerate((33, 2, 1, 1, 30)):
        (_, pos, par), _ = _params([size, 3], [at, 0], slots=[2, 0])
        rows = torch.cat([proj[at:at + size], proj[:3]]).to(DEV)
        # the last portion runs as chunks of 7 tokens side by side (3 of the second sequence's tokens fill less than one)
        o = kernels.mingru_scan(rows, bz.to(DEV), bx.to(DEV), state, par.q_cu_seq_lens, pos, par.state_slots, 2, width,
                                q_max=size, chunk_len=7 if k == 4 else 0)
        got.append(o[:size].float().cpu())
        assert float((o[size:].cpu().double() - ref[:3]).abs().max()) < tol
        at += size
    assert float((torch.cat(got).double() - ref).abs().max()) < tol
    assert float((state[2].cpu().double() - S).abs().max()) < 1e-5 and float(state[1].min()) == 7.0


def _attend_case(dtype, H, G, dim, vdim, window, keep, block_size, cached, n_new, loud, seed=0, n_splits=0):
    """The attention kernel alone over a hand-made cache: the first map's query of row i points along key `loud[i]`,
    so that this key (if it is visible) takes most of the row's weight in that map.  Returns (got, want)."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(seed)
    n = cached + n_new
    K = torch.randn(n, G, 2, dim, generator=g)
    V = torch.randn(n, G, vdim, generator=g)
    q = torch.randn(n_new, H, 2, dim, generator=g)
    pos = torch.arange(cached, n)
    for i, j in enumerate(loud):
        if j is None:
            continue
        for hh in range(H):
            q[i, hh, 0] = 6.0 * K[j, hh // (H // G), 0] / K[j, hh // (H // G), 0].norm()
    K, V = K.to(dtype), V.to(dtype)
    (_, _, par), hb = _params([n_new], [cached], block_size=block_size)
    slots_all = []
    table = hb.block_tables
    for j in range(n):
        slots_all.append(int(table[j // block_size]) + j % block_size)
    kc = torch.zeros(256 * block_size, G, 2 * dim, dtype=dtype)
    vc = torch.zeros(256 * block_size, G, vdim, dtype=dtype)
    kc[slots_all] = K.reshape(n, G, 2 * dim)
    vc[slots_all] = V
    gate = torch.randn(n_new, H, generator=g).to(dtype)
    lam, diff, scale = 0.45, 0.3, 1.0 / math.sqrt(dim)
    got = kernels.diff_attn(q.to(DEV), kc.to(DEV), vc.to(DEV), gate.to(DEV), par.q_cu_seq_lens, par.kv_cu_seq_lens,
                            par.block_tables, par.cu_block_lens, par.token_seq, block_size, scale, window, keep, lam,
                            1.0 - diff, 1e-5, 1, n_new, cached + n_new, n_splits)   # prompt-sized bf16 cases take the tensor-core kernel
    mask = {"size": window, "keep_first": keep} if window else None
    want = op.diff_attend(q.double(), K.double(), V.double(), pos, scale, mask, lam, diff, 1e-5)
    want = want * torch.sigmoid(gate.double())[:, :, None]
    return got.float().cpu().reshape(n_new, H, vdim).double(), want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 16, 24), (3, 3, 20, 8), (2, 1, 64, 130), (8, 2, 48, 80), (2, 2, 64, 128),
                                          (3, 1, 32, 16), (6, 2, 128, 64), (16, 2, 16, 32), (2, 2, 8, 12), (5, 1, 8, 16), (34, 1, 16, 16), (4, 2, 128, 128), (2, 1, 64, 64),
                                          (4, 4, 32, 64), (4, 1, 32, 32)])
def test_attention_window_and_kept_tokens_edges(dtype, H, G, dim, vdim):
    """Decoded rows (one new token each) and prompt rows whose loud key lies just inside / just outside the window,
    on the last kept token / the first one not kept, and far back with no window at all."""
    window, keep, cached = 10, 3, 41
    tol = 1e-4 if dtype == torch.float32 else 0.05
    # rows at positions 41 .. 46: window of row i covers i - 9 .. i
    loud = [32, 32, 2, 3, 36, 0]       # window's last key, just outside it, last kept token, first not kept, edge, kept
    got, want = _attend_case(dtype, H, G, dim, vdim, window, keep, 4, cached, 6, loud, seed=dim)
    assert float((got - want).abs().max()) < tol
    # the loud key really decides the row where it is visible, and is really unseen where it is not
    for row, j in ((1, 32), (3, 3)):
        assert not op.visible(cached + row, j, {"size": window, "keep_first": keep})
    for row, j in ((0, 32), (2, 2), (4, 36), (5, 0)):
        assert op.visible(cached + row, j, {"size": window, "keep_first": keep})
    # one decoded token with everything cached, then the same without a window: key 1 of 300 decides
    for win, kp in ((10, 3), (0, 0), (7, 0)):
        for n_splits in (0, 1, 2, 3, 9):      # the row's key tiles shared out over several CTAs, some left empty
            got, want = _attend_case(dtype, H, G, dim, vdim, win, kp, 8, 300, 1, [1], seed=7, n_splits=n_splits)
            assert float((got - want).abs().max()) < tol, (win, kp, n_splits)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_first_tokens_and_block_borders(dtype):
    tol = 1e-4 if dtype == torch.float32 else 0.05
    # a prompt from position 0: rows shorter than the window, shorter than the kept tokens, and block size 1 / 3 / 16
    for bs in (1, 3, 16):
        for vdim in (24, 32):       # CUDA-core and (bf16) tensor-core kernel
            got, want = _attend_case(dtype, 4, 2, 16, vdim, 5, 2, bs, 0, 19,
                                     [0, 0, 1, 2, 3, 1, 2, 2, None, 4, 6, 7, 1, 9, 9, None, 0, 13, 18], seed=bs)
            assert float((got - want).abs().max()) < tol
    # long portions on top of a long cache: key tiles that hold kept tokens only, the window's first tile, tile borders
    for win, kp, cached, n_new in ((40, 35, 100, 70), (33, 0, 31, 97), (0, 0, 64, 64), (64, 70, 200, 33), (200, 3, 5, 130)):
        loud = [None] * n_new
        loud[0], loud[-1], loud[n_new // 2] = max(0, cached - win + 1) if win else 0, kp - 1 if kp else cached, 0
        got, want = _attend_case(dtype, 4, 2, 32, 48, win, kp, 16, cached, n_new, loud, seed=win + kp)
        assert float((got - want).abs().max()) < tol, (win, kp, cached, n_new)
    # two new tokens (the single-token kernels) on caches that end just before, at and just after a 64-key tile border
    for cached in (0, 1, 62, 63, 64, 65, 127, 128, 200):
        for H, G in ((8, 2), (3, 3)):
            got, want = _attend_case(dtype, H, G, 32, 48, 50, 5, 16, cached, 2, [min(cached, 4), None], seed=cached)
            assert float((got - want).abs().max()) < tol, (cached, H, G)
    # window as long as, and longer than, the sequence; more kept tokens than the sequence has
    for win, kp in ((19, 0), (64, 0), (3, 40)):
        got, want = _attend_case(dtype, 2, 2, 8, 8, win, kp, 4, 0, 19, [None] * 19, seed=win)
        assert float((got - want).abs().max()) < tol


# ------------------------------------------------------------------ the model
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(pc.CONFIGS))
def test_whole_prompt_layers_and_logits(name, dtype):
    cfg = pc.CONFIGS[name]
    model, oracle = build(cfg, dtype)
    eng = engine_for(model)
    tokens = toks(75, cfg["vocab"], 1)
    lo = []
    want = oracle.forward(tokens, oracle.new_state(), lo)
    from scalellm_b200.decode_step import build_step_batch
    s = eng.open("x")
    eng.pool.reserve(s.seq, len(tokens))
    hb = build_step_batch(eng.pool, [s.seq], [tokens], [0], [s.slot], [-1])
    tok, pos, par = eng.bufs.upload(hb)
    got_layers = []
    got = model.forward(tok, pos, par, layer_out=got_layers)
    for a, b in zip(got_layers, lo):
        assert float((a.cpu().double() - b).abs().max()) < (2e-4 if dtype == torch.float32 else 0.05) * float(b.abs().max())
    assert pc.logits_error(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(pc.CONFIGS))
def test_prefill_decode_and_portions_agree_with_the_oracle(name, dtype):
    cfg = pc.CONFIGS[name]
    model, oracle = build(cfg, dtype, seed=1)
    tokens = toks(90, cfg["vocab"], 2)
    want = oracle_logits(oracle, tokens)
    for cuts in ([90], [58], [1] * 3, [2, 2, 5, 2, 31, 1, 2, 17, 2], [7] * 13, [33, 4, 4, 4, 40]):
        eng = engine_for(model, block_size=4)
        got = run_schedule(eng, tokens, cuts)
        assert pc.logits_error(got, want) < TOL[dtype], cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_portions_run_in_chunks(dtype):
    """Portions long enough for the chunked recurrence and for many key tiles, cut at places that are no multiple of
    the chunk or the tile, against the whole prompt in one step and the oracle."""
    cfg = pc.CONFIGS["mix"]
    model, oracle = build(cfg, dtype, seed=6)
    tokens = toks(333, cfg["vocab"], 7)
    want = oracle_logits(oracle, tokens)
    for cuts in ([333], [150, 2, 181], [129, 130, 71]):
        eng = engine_for(model, max_tokens=400, block_size=16)
        got = run_schedule(eng, tokens, cuts)
        assert pc.logits_error(got, want) < TOL[dtype], cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_batches_with_reused_blocks_and_slots(dtype):
    """Five unequal requests through a pool with room for three and three state slots: portions beside single
    tokens, requests that pause, blocks and slots handed on without being cleared."""
    from scalellm_b200.engine import StepEntry
    cfg = pc.CONFIGS["mix"]
    model, oracle = build(cfg, dtype, seed=2, max_seqs=3)
    lens = {"a": 61, "b": 9, "c": 40, "d": 1, "e": 33}
    T = {k: toks(n, cfg["vocab"], 10 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: oracle_logits(oracle, v) for k, v in T.items()}
    eng = engine_for(model, max_tokens=128, block_size=4, max_seqs=3)
    plan = [[("a", 17), ("b", 2)], [("a", 2), ("b", 1), ("c", 5)], [("b", 6), ("c", 1)], [("a", 30), ("c", 30)],
            [("a", 1), ("c", 2)], [("a", 1), ("c", 2), ("d", 1)], [("a", 10), ("e", 2)], [("e", 29)], [("e", 1)], [("e", 1)]]
    at = {k: 0 for k in T}
    got = {k: [] for k in T}
    for step in plan:
        entries = [StepEntry(k, T[k][at[k]:at[k] + n], list(range(n))) for k, n in step]
        out = eng.step(entries).float().cpu()
        r = 0
        for k, n in step:
            got[k].append(out[r:r + n])
            r += n
            at[k] += n
            if at[k] == lens[k]:
                eng.finish(k)
    for k in T:
        assert at[k] == lens[k]
        assert pc.logits_error(torch.cat(got[k]), want[k]) < TOL[dtype], k


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_small_blocks(dtype):
    cfg = pc.CONFIGS["attn_first"]
    model, oracle = build(cfg, dtype, seed=3)
    tokens = toks(150, cfg["vocab"], 4)
    want = oracle_logits(oracle, tokens)
    eng = engine_for(model, max_tokens=160, block_size=2)
    got = run_schedule(eng, tokens, [3])
    assert pc.logits_error(got, want) < TOL[dtype]


def test_graph_replay_of_single_token_steps():
    cfg = pc.CONFIGS["mix"]
    model, oracle = build(cfg, torch.bfloat16, seed=4)
    tokens = toks(40, cfg["vocab"], 5)
    want = oracle_logits(oracle, tokens)
    eng = engine_for(model, block_size=4, use_graphs=True)
    got = run_schedule(eng, tokens, [6])
    assert eng._graphs, "no graph was captured"
    assert pc.logits_error(got, want) < TOL[torch.bfloat16]


def test_greedy_generation_through_the_scheduler():
    """More requests than places; the ids must be those of greedy decoding with the oracle wherever its two
    best logits are not a near tie."""
    from scalellm_b200.engine import SamplingParams
    cfg = pc.CONFIGS["plain"]
    model, oracle = build(cfg, torch.float32, seed=5, max_seqs=2)
    eng = engine_for(model, max_tokens=96, block_size=4, max_seqs=2)
    prompts = [toks(n, cfg["vocab"], 20 + n) for n in (5, 17, 1, 9)]
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=6) for _ in prompts], max_step_tokens=8)
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        st = oracle.new_state()
        lg = oracle.forward(p, st)[-1]
        for tok in o:
            top = torch.topk(lg, 2).values
            if float(top[0] - top[1]) > 1e-3:
                assert int(lg.argmax()) == tok
            lg = oracle.forward([tok], st)[-1]
