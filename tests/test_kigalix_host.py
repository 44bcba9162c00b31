"""CPU: host-side pieces of the Kigalix path — the restatement's own consistency, the shape table, the
checkpoint reader, block and state-slot reuse, step metadata, the scheduler's budget logic, the registry."""
import os

import numpy as np
import pytest
import torch

from oracle import kigalix as ok
from tests import kigalix_case as kc


def test_restatement_whole_equals_token_by_token():
    cfg = kc.CONFIGS["mix"]
    o = ok.Kigalix(cfg, kc.weights(cfg, 3))
    tokens = [int(x) for x in np.random.default_rng(0).integers(0, cfg["vocab"], 30)]
    whole = o.forward(tokens, o.new_state())
    st, parts = o.new_state(), []
    for cut in ([tokens[:7]], [tokens[7:9]], [[t] for t in tokens[9:]]):
        for piece in cut:
            parts.append(o.forward(piece, st))
    assert float((torch.cat(parts) - whole).abs().max()) < 1e-9


def test_rotary_tables_match_the_restatement():
    from scalellm_b200.kigalix import rotary_table
    for rot in ({"base": 10000.0, "dims": 16}, {"base": 500000.0, "dims": 64,
                                               "scaling": {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}},
                {"base": 1e6, "dims": 24, "scaling": {"factor": 3.0, "original": 100, "fast": 9.0, "slow": 2.0}}):
        f, m = rotary_table(rot)
        rf, rm = ok.rope_table(rot)
        assert float((f.double() / rf - 1).abs().max()) < 1e-7 and abs(m - rm) < 1e-12


def test_shape_table_matches_the_tests_own():
    from scalellm_b200.kigalix import tensor_shapes
    for cfg in kc.CONFIGS.values():
        mine, theirs = kc.shapes(cfg, decay_rank=16), tensor_shapes(cfg)
        assert {k: tuple(v) for k, v in theirs.items()} == mine


def test_checkpoint_round_trip(tmp_path):
    from scalellm_b200 import checkpoint
    t = {"a.b": torch.randn(3, 5).to(torch.bfloat16), "n": torch.arange(7, dtype=torch.int32), "f": torch.randn(2, 2, 2)}
    path = os.path.join(tmp_path, "model.safetensors")
    checkpoint.write_safetensors(path, t)
    back = checkpoint.read_safetensors(path)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    same = ok.read_safetensors(path)                 # the restatement's own reader agrees
    assert all(torch.equal(same[k], t[k]) for k in t)


def test_blocks_and_slots_are_used_again():
    from scalellm_b200.decode_step import BlockPool, StateSlotPool
    pool = BlockPool(10, 4, seed=1)
    a, b = pool.open_sequence(), pool.open_sequence()
    pool.reserve(a, 9)
    pool.reserve(b, 16)
    assert len(pool.seq_blocks[a]) == 3 and len(pool.seq_blocks[b]) == 4 and pool.n_free_blocks() == 3
    pool.reserve(a, 12)                               # already has them
    assert pool.n_free_blocks() == 3
    with pytest.raises(RuntimeError):
        pool.reserve(a, 29)
    old = set(pool.seq_blocks[a])
    pool.release(a)
    c = pool.open_sequence()
    assert c == a and pool.n_free_blocks() == 6
    pool.reserve(c, 24)
    assert old <= set(pool.seq_blocks[c]) and pool.n_free_blocks() == 0
    assert set(pool.seq_blocks[c]).isdisjoint(pool.seq_blocks[b])
    slots = StateSlotPool(2)
    x, y = slots.take(), slots.take()
    with pytest.raises(RuntimeError):
        slots.take()
    slots.give_back(x)
    assert slots.take() == x and {x, y} == {0, 1}


def test_step_metadata_of_portions_and_decodes():
    from scalellm_b200.decode_step import BlockPool, build_step_batch
    pool = BlockPool(32, 4, seed=5)
    s0, s1, s2 = (pool.open_sequence() for _ in range(3))
    pool.reserve(s0, 11)
    pool.reserve(s1, 3)
    pool.reserve(s2, 8)
    hb = build_step_batch(pool, [s2, s0, s1], [[5, 6, 7], [9], [1, 2, 3]], [5, 10, 0], [2, 0, 1])
    assert hb.tokens.tolist() == [5, 6, 7, 9, 1, 2, 3]
    assert hb.positions.tolist() == [5, 6, 7, 10, 0, 1, 2]
    assert hb.q_cu_lens.tolist() == [0, 3, 4, 7] and hb.kv_cu_lens.tolist() == [0, 8, 19, 22]
    assert hb.token_seq.tolist() == [0, 0, 0, 1, 2, 2, 2] and hb.state_slots.tolist() == [2, 0, 1]
    assert hb.cu_block_lens.tolist() == [0, 2, 5, 6]
    tab = hb.block_tables.tolist()
    assert tab[0:2] == [b * 4 for b in pool.seq_blocks[s2][:2]] and tab[2:5] == [b * 4 for b in pool.seq_blocks[s0][:3]]
    assert hb.new_cache_slots.tolist()[3] == pool.seq_blocks[s0][2] * 4 + 2
    assert hb.new_cache_slots.tolist()[0] == pool.seq_blocks[s2][1] * 4 + 1


class _FakeModel:
    needs_state_slots, n_vocab, dtype, device = True, 11, torch.float32, torch.device("cpu")

    def alloc_cache(self, n_blocks, block_size):
        pass

    def forward(self, tokens, positions, params, last_token_idxes=None):
        """Logits that make greedy sampling return (token + position) % vocab."""
        nxt = (tokens.long() + positions.long()) % self.n_vocab
        return torch.nn.functional.one_hot(nxt, self.n_vocab).float().index_select(0, last_token_idxes.long())


def test_scheduler_budget_decodes_first_and_admission(monkeypatch):
    from scalellm_b200 import engine as E
    monkeypatch.setattr(E.Sampler, "__call__", lambda self, lg, seqs: [int(x) for x in lg.argmax(-1)])
    eng = E.Engine(_FakeModel(), max_tokens=64, block_size=4, max_seqs=2)
    sched = E.Scheduler(eng, 8)
    sched.add("p", list(range(13)), E.SamplingParams(max_new_tokens=3))
    sched.add("q", [4, 4, 4], E.SamplingParams(max_new_tokens=2))
    sched.add("r", [1], E.SamplingParams(max_new_tokens=1))
    e1 = sched.next_step()
    assert [(e.rid, len(e.tokens), e.want) for e in e1] == [("p", 8, [])] and len(sched.waiting) == 1
    eng.step(e1)
    e2 = sched.next_step()
    assert [(e.rid, len(e.tokens), e.want) for e in e2] == [("p", 5, [4]), ("q", 3, [2])]
    eng2 = E.Engine(_FakeModel(), max_tokens=64, block_size=4, max_seqs=2)
    got = eng2.generate([[3, 0, 0, 2], [5], [1, 1]], [E.SamplingParams(max_new_tokens=n) for n in (3, 2, 4)],
                        max_step_tokens=3)
    def expect(prompt, n):
        seq, out = list(prompt), []
        for _ in range(n):
            out.append((seq[-1] + len(seq) - 1) % 11)
            seq.append(out[-1])
        return out
    assert got == [expect([3, 0, 0, 2], 3), expect([5], 2), expect([1, 1], 4)]
    assert eng2.pool.n_free_blocks() == 16 and len(eng2.slots.free) == 2 and not eng2.seqs


def test_registry_reads_the_architecture():
    from scalellm_b200 import registry
    from scalellm_b200.kigalix import KigalixDecoder
    assert registry.model_class({"architecture": "Kigalix"}) is KigalixDecoder
    assert registry.architecture_of({"architectures": ["LlamaForCausalLM"]}) == "LlamaForCausalLM"
    with pytest.raises(ValueError):
        registry.model_class({"architecture": "NoSuchModel"})
