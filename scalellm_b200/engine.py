"""Serving engine: requests, continuous batching with chunked prefill, the step function, sampling.

The reference splits this over its scheduler (src/scheduler/continuous_scheduler.cpp: a token budget per
step, decodes first, then prompt portions), its block manager (src/memory/block_manager.cpp) and its
engine / worker (src/engine/llm_engine.cpp, worker.cpp: prepare inputs, run the model, sample).  Here:

    Engine.step(entries)   the step function: any mix of prompt portions and single decoded tokens of
                           live sequences in ONE packed batch -> logits of the asked rows.  Blocks are
                           taken from the BlockPool as sequences grow, state slots from the StateSlotPool;
                           Engine.finish() gives both back, so pages and slots are used again.
    Scheduler              which sequences run next and with how many tokens (token budget per step).
    Sampler                greedy argmax, or temperature / top-k / top-p through the logits-processor kernels.
    Engine.generate()      the loop a user calls: prompts (token ids) in, generated ids out.

`bin/trace_run` replays a given schedule through Engine.step; generate() lets the Scheduler make one.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib, kernels
from .decode_step import BlockPool, StateSlotPool, StepBuffers, build_step_batch


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 0.0          # 0: greedy
    top_k: int = 0                    # 0: off
    top_p: float = 1.0                # >= 1: off
    seed: int = 0


@dataclass
class Sequence_:
    rid: str
    seq: int                          # index in the BlockPool
    slot: int                         # state slot (-1: the model keeps no recurrent state)
    n_cached: int = 0                 # tokens already run
    last_token: int = -1              # the last token run (-1: none yet); embeddings that read the token before use it
    prompt: List[int] = field(default_factory=list)
    output: List[int] = field(default_factory=list)
    sampling: SamplingParams = field(default_factory=SamplingParams)


@dataclass
class StepEntry:
    rid: str
    tokens: List[int]
    want: List[int] = field(default_factory=list)    # rows (within tokens) whose logits are returned


class Sampler:
    """Next-token choice from logits rows [n, vocab]."""

    def __init__(self, device):
        self.device = device
        self._gen: Dict[str, torch.Generator] = {}

    def __call__(self, logits: torch.Tensor, seqs: List[Sequence_]) -> List[int]:
        if all(s.sampling.temperature <= 0.0 for s in seqs):
            _lib.ensure(("elementwise.cu",))
            return [int(x) for x in kernels.argmax(logits.contiguous()).tolist()]
        _lib.ensure(("elementwise.cu", "sampling.cu"))
        lg = logits.to(torch.bfloat16).clone().contiguous()   # the logits processors work in place, in 16 bits
        greedy = kernels.argmax(lg)
        temps = torch.tensor([max(s.sampling.temperature, 1e-6) for s in seqs], dtype=torch.float32,
                             device=self.device).to(lg.dtype)
        kernels.apply_temperature_penalty(lg, temps)
        top_k = torch.tensor([s.sampling.top_k for s in seqs], dtype=torch.int64, device=self.device)
        top_p = torch.tensor([s.sampling.top_p for s in seqs], dtype=torch.float32, device=self.device)
        kernels.apply_top_k_top_p(lg, top_k, top_p)
        kernels.invoke_softmax(lg)
        out = []
        for i, s in enumerate(seqs):
            if s.sampling.temperature <= 0.0:
                out.append(int(greedy[i]))
                continue
            g = self._gen.get(s.rid)
            if g is None:
                g = self._gen[s.rid] = torch.Generator(device=self.device).manual_seed(s.sampling.seed)
            out.append(int(torch.multinomial(lg[i].float(), 1, generator=g)))
        return out

    def forget(self, rid: str) -> None:
        self._gen.pop(rid, None)


class Scheduler:
    """Continuous batching under a token budget: every running sequence that has finished its prompt gets
    its one decode token first; what is left of the budget goes to prompt portions in arrival order, and
    waiting requests are admitted while sequence places, state slots and blocks last."""

    def __init__(self, engine: "Engine", max_step_tokens: int):
        self.engine, self.max_step_tokens = engine, max_step_tokens
        self.waiting: Deque[Tuple[str, List[int], SamplingParams]] = deque()
        self.running: List[Sequence_] = []

    def add(self, rid: str, prompt: Sequence[int], sampling: SamplingParams) -> None:
        if not prompt:
            raise ValueError("empty prompt")
        self.waiting.append((rid, list(prompt), sampling))

    def _admit(self) -> None:
        eng = self.engine
        while self.waiting and len(self.running) < eng.max_seqs:
            rid, prompt, sp = self.waiting[0]
            need = -(-(len(prompt) + sp.max_new_tokens) // eng.pool.block_size)
            held = sum(-(-(len(s.prompt) + s.sampling.max_new_tokens) // eng.pool.block_size)
                       - len(eng.pool.seq_blocks[s.seq]) for s in self.running)
            if need + held > eng.pool.n_free_blocks():
                if not self.running:
                    raise RuntimeError(f"request {rid} needs {need} blocks; the pool has {eng.pool.n_free_blocks()}")
                break
            self.waiting.popleft()
            s = eng.open(rid)
            s.prompt, s.sampling = prompt, sp
            self.running.append(s)

    def next_step(self) -> List[StepEntry]:
        self._admit()
        budget, entries = self.max_step_tokens, []
        for s in self.running:                      # decodes
            if s.n_cached >= len(s.prompt) and budget > 0:
                entries.append(StepEntry(s.rid, [s.output[-1]], [0]))
                budget -= 1
        for s in self.running:                      # prompt portions
            left = len(s.prompt) - s.n_cached
            if left > 0 and budget > 0:
                n = min(left, budget)
                toks = s.prompt[s.n_cached: s.n_cached + n]
                entries.append(StepEntry(s.rid, toks, [n - 1] if n == left else []))
                budget -= n
        return entries

    def done(self) -> bool:
        return not self.waiting and not self.running


class Engine:
    def __init__(self, model, max_tokens: int, block_size: int = 16, max_seqs: int = 4,
                 max_step_tokens: Optional[int] = None, pool_seed: int = 2, use_graphs: bool = False):
        """max_tokens: tokens the cache pool holds at any time, each sequence rounded up to whole blocks.
        use_graphs: steps in which every sequence brings one token (decoding) replay a CUDA graph, captured
        per batch size and power-of-two bucket of the longest cached length once such a step has run twice
        eagerly (the eager runs create the workspaces and library handles a capture must not create; a
        warm-up run of its own would advance the recurrent state twice)."""
        self.model, self.max_seqs = model, max_seqs
        self.device = model.device
        n_blocks = -(-max_tokens // block_size)
        self.pool = BlockPool(n_blocks, block_size, seed=pool_seed)
        self.slots = StateSlotPool(max_seqs) if getattr(model, "needs_state_slots", False) else None
        model.alloc_cache(n_blocks, block_size)
        self.max_step_tokens = max_step_tokens or n_blocks * block_size
        self.needs_prev = bool(getattr(model, "needs_prev_token", False))
        self.bufs = StepBuffers(self.device, self.max_step_tokens, max_seqs, n_blocks + max_seqs, self.needs_prev)
        self.seqs: Dict[str, Sequence_] = {}
        self.sampler = Sampler(self.device)
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self._graphs: Dict[Tuple[int, int], Tuple[torch.cuda.CUDAGraph, torch.Tensor]] = {}
        self._seen: Dict[Tuple[int, int], int] = {}

    # ---------------------------------------------------------------- sequences
    def open(self, rid: str) -> Sequence_:
        if rid in self.seqs:
            raise KeyError(f"request {rid} is live already")
        if len(self.seqs) >= self.max_seqs:
            raise RuntimeError("no place for another sequence")
        s = Sequence_(rid, self.pool.open_sequence(), self.slots.take() if self.slots else -1)
        self.seqs[rid] = s
        return s

    def finish(self, rid: str) -> None:
        s = self.seqs.pop(rid)
        self.pool.release(s.seq)
        if self.slots:
            self.slots.give_back(s.slot)
        self.sampler.forget(rid)

    # ---------------------------------------------------------------- the step function
    def step(self, entries: List[StepEntry]) -> torch.Tensor:
        """Runs the entries' tokens as one batch on top of what earlier steps left in the cache and state;
        a request not seen before is admitted.  Returns logits [sum of len(want), vocab] in entry order."""
        entries = [e for e in entries if e.tokens]
        if not entries:
            return torch.empty((0, self.model.n_vocab), dtype=self.model.dtype, device=self.device)
        seqs = [self.seqs.get(e.rid) or self.open(e.rid) for e in entries]
        if len({s.rid for s in seqs}) != len(seqs):
            raise ValueError("a request appears twice in one step")
        want, row0 = [], 0
        for e, s in zip(entries, seqs):
            self.pool.reserve(s.seq, s.n_cached + len(e.tokens))
            want += [row0 + int(w) for w in e.want]
            row0 += len(e.tokens)
        if row0 > self.max_step_tokens:
            raise ValueError(f"{row0} tokens in one step; the engine was made for {self.max_step_tokens}")
        hb = build_step_batch(self.pool, [s.seq for s in seqs], [e.tokens for e in entries],
                              [s.n_cached for s in seqs], [s.slot for s in seqs] if self.slots else None,
                              [s.last_token for s in seqs] if self.needs_prev else None)
        idx = torch.tensor(want, dtype=torch.int32).to(self.device, non_blocking=True)
        if self.use_graphs and row0 == len(entries):
            logits = self._decode_step(hb, idx, want)
        else:
            tokens, positions, params = self.bufs.upload(hb)
            logits = self.model.forward(tokens, positions, params, last_token_idxes=idx)
        for e, s in zip(entries, seqs):
            s.n_cached += len(e.tokens)
            s.last_token = int(e.tokens[-1])
        return logits

    def _decode_step(self, hb, idx: torch.Tensor, want: List[int]) -> torch.Tensor:
        """One token per sequence: replay (or, the third time round, capture) the step's CUDA graph."""
        B = len(hb.q_cu_lens) - 1
        bucket = 256
        while bucket < hb.kv_max:
            bucket *= 2
        key = (B, bucket)
        hb.kv_max = bucket            # an upper bound: it sizes work partitions, the lengths come from the device
        tokens, positions, params = self.bufs.upload(hb)
        if key not in self._graphs:
            self._seen[key] = self._seen.get(key, 0) + 1
            if self._seen[key] <= 2:
                return self.model.forward(tokens, positions, params, last_token_idxes=idx)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self.model.forward(tokens, positions, params)
            self._graphs[key] = (graph, out)
        graph, out = self._graphs[key]
        graph.replay()
        return out if want == list(range(B)) else out.index_select(0, idx)

    # ---------------------------------------------------------------- generation
    def generate(self, prompts: Sequence[Sequence[int]], sampling: Optional[Sequence[SamplingParams]] = None,
                 max_step_tokens: Optional[int] = None, eos: Optional[int] = None) -> List[List[int]]:
        """Token ids in, generated token ids out (one list per prompt, in order)."""
        sampling = list(sampling) if sampling is not None else [SamplingParams() for _ in prompts]
        sched = Scheduler(self, min(max_step_tokens or self.max_step_tokens, self.max_step_tokens))
        for i, (p, sp) in enumerate(zip(prompts, sampling)):
            sched.add(f"g{i}", p, sp)
        results: Dict[str, List[int]] = {}
        while not sched.done():
            entries = sched.next_step()
            if not entries:
                raise RuntimeError("the scheduler made an empty step with work left")
            logits = self.step(entries)
            asked = [self.seqs[e.rid] for e in entries if e.want]
            if asked:
                for s, tok in zip(asked, self.sampler(logits, asked)):
                    s.output.append(tok)
            for s in list(sched.running):
                if s.n_cached >= len(s.prompt) and (len(s.output) >= s.sampling.max_new_tokens
                                                    or (eos is not None and s.output and s.output[-1] == eos)):
                    results[s.rid] = s.output
                    sched.running.remove(s)
                    self.finish(s.rid)
        return [results[f"g{i}"] for i in range(len(prompts))]
