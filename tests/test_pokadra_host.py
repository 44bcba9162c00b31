"""CPU: host-side parts of the Pokadra path — the plain restatement against itself (whole prompt, token by token,
portions), the product's shape table and rotary table against the tests' own, the previous-token column of a
step's metadata, the registry."""
import math

import numpy as np
import torch

from oracle import pokadra as op
from tests import pokadra_case as pc


def toks(n, vocab, seed):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, size=n)]


def test_oracle_whole_equals_token_by_token_and_portions():
    for name, cfg in pc.CONFIGS.items():
        m = op.Pokadra(cfg, pc.weights(cfg, 1))
        tokens = toks(40, cfg["vocab"], 3)
        whole = m.forward(tokens, m.new_state())
        st, rows = m.new_state(), []
        for t in tokens:
            rows.append(m.forward([t], st))
        assert float((torch.cat(rows) - whole).abs().max()) < 1e-9, name
        st, rows, at = m.new_state(), [], 0
        for n in (7, 2, 1, 19, 11):
            rows.append(m.forward(tokens[at:at + n], st))
            at += n
        assert float((torch.cat(rows) - whole).abs().max()) < 1e-9, name


def test_oracle_mechanisms_by_hand():
    # the window: position 12 with size 4 and two kept tokens sees 0, 1 and 9 .. 12
    mask = {"size": 4, "keep_first": 2}
    assert [j for j in range(20) if op.visible(12, j, mask)] == [0, 1, 9, 10, 11, 12]
    assert [j for j in range(5) if op.visible(2, j, mask)] == [0, 1, 2]
    assert [j for j in range(5) if op.visible(3, j, None)] == [0, 1, 2, 3]
    # group norm: every group has unit mean square before the weight
    y = torch.randn(3, 12, dtype=torch.float64) * torch.tensor([1.0] * 4 + [50.0] * 4 + [0.01] * 4)
    n = op.group_norm(y, torch.ones(12, dtype=torch.float64), 3, 0.0)
    assert torch.allclose(n.reshape(3, 3, 4).pow(2).mean(-1), torch.ones(3, 3, dtype=torch.float64))
    # the candidate is continuous at zero and positive
    u = torch.tensor([-1e-9, 0.0, 1e-9, -30.0], dtype=torch.float64)
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    assert float((c[:3] - 0.5).abs().max()) < 1e-8 and float(c[3]) > 0.0
    # rotation keeps the length of every rotated pair up to the multiplier and leaves the rest alone
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 8.0, "original": 32, "fast": 8.0, "slow": 2.0}}
    x = torch.randn(5, 2, 6, dtype=torch.float64)
    r = op.rotate(x, torch.arange(5), rot)
    mult = 0.1 * math.log(8.0) + 1.0
    assert torch.allclose(r[..., :4].reshape(5, 2, 2, 2).norm(dim=-1), mult * x[..., :4].reshape(5, 2, 2, 2).norm(dim=-1))
    assert torch.equal(r[..., 4:], x[..., 4:])
    # the pair table: the last row at a sequence's start, the hashed row after
    w = {"embed": torch.zeros(10, 3, dtype=torch.float64), "bigram": torch.arange(8, dtype=torch.float64)[:, None].expand(8, 3)}
    e = op.embedding([4, 9], None, w, {"scale": 1.0, "bigram": {"buckets": 7, "mul_prev": 5, "mul_cur": 3}})
    assert float(e[0, 0]) == 7.0 and float(e[1, 0]) == float((4 * 5 + 9 * 3) % 7)


def test_shape_table_and_random_weights():
    from scalellm_b200 import pokadra
    for name, cfg in pc.CONFIGS.items():
        assert pokadra.tensor_shapes(cfg) == pc.shapes(cfg), name
        w = pokadra.random_tensors(cfg, 0)
        assert {k: tuple(v.shape) for k, v in w.items()} == pc.shapes(cfg)


def test_rotary_table_matches_the_restatement():
    from scalellm_b200 import pokadra
    for rot in ({"base": 10000.0, "dims": 8}, {"base": 500.0, "dims": 16, "scaling": {"factor": 8.0, "original": 32, "fast": 8.0, "slow": 2.0}},
                {"base": 1e6, "dims": 64, "scaling": {"factor": 2.5, "original": 4096, "fast": 32.0, "slow": 1.0}}):
        f, mult, dims = pokadra.rotary_table(rot)
        rf, rmult = op.rotary_frequencies(rot)
        assert dims == rot["dims"] and abs(mult - rmult) < 1e-12
        assert float((f.double() - rf).abs().max() / rf.abs().max()) < 1e-7
    assert pokadra.rotary_table(None) == (None, 1.0, 0)


def test_step_metadata_carries_the_previous_token():
    from scalellm_b200.decode_step import BlockPool, StepBuffers, build_step_batch
    pool = BlockPool(16, 4, seed=0)
    seqs = [pool.open_sequence() for _ in range(3)]
    for s, n in zip(seqs, (5, 9, 1)):
        pool.reserve(s, n)
    hb = build_step_batch(pool, seqs, [[3, 4, 5], [8], [6]], [2, 8, 0], [0, 1, 2], [11, 12, -1])
    assert hb.prev_tokens.tolist() == [11, 3, 4, 12, -1]
    assert build_step_batch(pool, seqs, [[3, 4, 5], [8], [6]], [2, 8, 0], [0, 1, 2]).prev_tokens is None
    dev = torch.device("cpu")
    plain, with_prev = StepBuffers(dev, 32, 4, 20), StepBuffers(dev, 32, 4, 20, with_prev_tokens=True)
    assert with_prev.total == plain.total + 32          # models that do not ask for it copy what they did before
    tok, pos, par = with_prev.upload(hb)
    assert par.prev_tokens.tolist() == [11, 3, 4, 12, -1] and plain.upload(hb)[2].prev_tokens is None


def test_engine_remembers_the_last_token():
    """A fake model records the step's previous-token column: portions, a pause and a reused place."""
    from scalellm_b200.engine import Engine, StepEntry

    class Fake:
        needs_state_slots, needs_prev_token, n_vocab, dtype = True, True, 5, torch.float32
        device = torch.device("cpu")
        seen = []

        def alloc_cache(self, n_blocks, block_size):
            pass

        def forward(self, tokens, positions, params, last_token_idxes=None):
            self.seen.append(params.prev_tokens.tolist())
            return torch.zeros((len(last_token_idxes), 5))

    m = Fake()
    eng = Engine(m, 64, block_size=4, max_seqs=2)
    eng.step([StepEntry("a", [1, 2, 3], []), StepEntry("b", [7], [])])
    eng.step([StepEntry("b", [8, 9], [])])
    eng.step([StepEntry("a", [4], []), StepEntry("b", [3], [])])
    eng.finish("a")
    eng.step([StepEntry("c", [5, 5], [])])
    assert m.seen == [[-1, 1, 2, -1], [7, 8], [3, 9], [-1, 5]]


def test_registry_knows_the_architecture():
    from scalellm_b200 import registry
    from scalellm_b200.pokadra import PokadraDecoder
    assert registry.model_class({"architecture": "Pokadra"}) is PokadraDecoder
    assert registry.model_class({"architecture": "pokadra"}) is PokadraDecoder
