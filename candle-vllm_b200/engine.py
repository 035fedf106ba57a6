"""Serving loop for ragged-step models: the step function (``ModelRunner.execute``), the request scheduler with chunked prefill and
continuous batching, and ``LLMEngine.generate``.  Roles follow the reference's ``LLMEngine`` + ``Scheduler``
(src/openai/pipelines/llm_engine.rs, src/scheduler/mod.rs): waiting -> running queues, a token budget per
step, blocks from ``BlockManager``, recurrent-state slots from ``StateCache``; unlike the reference a step may carry prompt portions
and decoded tokens together.

``ModelRunner`` is the only place that touches caches: it owns the ``CacheEngine`` (paged K / V per attention run), the ``StateCache``
(f32 state per recurrent run) and the ``BlockManager``; callers name sequences by id.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ._lib import BackendError
from .block_manager import BlockManager
from .cache_engine import CacheConfig, CacheEngine
from .inputs import prepare_step
from .sampling import Sampler, SamplingParams
from .seq_ops import StepBatch
from .state_cache import StateCache


class _DecodeGraph:
    """A captured step of B single-token entries (the reference replays captured decode graphs the same way,
    src/backend/graph.rs:685-803): static metadata buffers, two small H2D copies and one graph launch per step.
    Warm-up runs on a scratch state slot with the cache write switched off, so capturing disturbs no live sequence."""

    def __init__(self, runner: "ModelRunner", B: int, width: int):
        dev = runner.model.device
        self.B, self.W = B, width
        n = B * (4 + width) + B + 1
        # two pinned staging sets used in turn: a set is rewritten only after the copy that last read it has run on the device
        self.stage = [(torch.zeros(n, dtype=torch.int32).pin_memory(), torch.zeros(B, dtype=torch.int64).pin_memory(), torch.cuda.Event()) for _ in range(2)]
        self.turn = 0
        self.meta = torch.zeros(n, dtype=torch.int32, device=dev)
        m = self.meta
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.batch = StepBatch(tokens=m[0:B], positions=m[B:2 * B], token_seq=ar[:B].clone(), slot_mapping=torch.full((B,), -1, dtype=torch.int64, device=dev),
                               cu_seqlens=ar, cu_seqlens_k=m[4 * B + B * width:], seq_slots=m[2 * B:3 * B], seq_start=m[3 * B:4 * B],
                               block_tables=m[4 * B:4 * B + B * width].view(B, width),
                               want_rows=ar[:B].clone(), num_tokens=B, num_seqs=B, num_want=B, max_position=0, pure_decode=True)
        self.meta[2 * B:3 * B] = runner.state.scratch_slot
        self.meta[4 * B + B * width:] = ar                     # warm-up: one key per entry
        kv = runner.cache.gpu_cache if runner.cache else []
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                runner.model.forward(self.batch, kv, runner.state.tensors)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = runner.model.forward(self.batch, kv, runner.state.tensors)

    def replay(self, prep: dict) -> torch.Tensor:
        host, host_slots, copied = self.stage[self.turn]
        self.turn ^= 1
        copied.synchronize()
        B, h = self.B, host.numpy()
        h[0:B], h[B:2 * B], h[2 * B:3 * B], h[3 * B:4 * B] = prep["tokens"], prep["positions"], prep["seq_slots"], prep["seq_start"]
        bt = prep["block_tables"]
        tab = h[4 * B:4 * B + B * self.W].reshape(B, self.W)
        tab[:, :bt.shape[1]] = bt
        h[4 * B + B * self.W:] = prep["cu_seqlens_k"]
        host_slots.numpy()[:] = prep["slot_mapping"]
        self.meta.copy_(host, non_blocking=True)
        self.batch.slot_mapping.copy_(host_slots, non_blocking=True)
        copied.record()
        self.graph.replay()
        return self.logits


class ModelRunner:
    def __init__(self, model, num_blocks: int, num_slots: int, block_size: int = 64, decode_graphs: bool = False, max_blocks_per_seq: int = 0):
        """``decode_graphs``: steps made of single tokens only (one wanted logit each) replay a CUDA graph captured per batch size;
        ``max_blocks_per_seq`` is the table width those graphs are captured with (default: the whole pool)."""
        self.model, self.block_size = model, block_size
        plan = model.cache_plan()
        kv = plan["kv_layers"]
        self.cache = CacheEngine(len(kv), 0, 0, CacheConfig(block_size, num_blocks), dtype=model.dtype, device=model.device, layer_shapes=kv,
                                 pool_shapes=plan.get("pool_layers")) if kv else None
        self.state = StateCache(plan["state_layers"], num_slots, device=model.device)
        self.blocks = BlockManager(block_size, num_blocks, 0)
        self.lengths: Dict[int, int] = {}          # tokens of each live sequence already in cache / state
        self.decode_graphs = decode_graphs
        self.graph_width = max_blocks_per_seq or num_blocks
        self._graphs: Dict[int, _DecodeGraph] = {}

    # -- sequence lifetime -------------------------------------------------------------------------------------------
    def can_admit(self, num_tokens: int, reserved_blocks: int = 0) -> bool:
        return self.state.pool.num_free() > 0 and -(-num_tokens // self.block_size) <= self.blocks.num_free_gpu_blocks() - reserved_blocks

    def admit(self, seq_id: int) -> None:
        if seq_id in self.lengths:
            raise BackendError(f"sequence {seq_id} is already live")
        self.state.pool.acquire(seq_id)
        self.lengths[seq_id] = 0

    def release(self, seq_id: int) -> None:
        self.blocks.free_table(seq_id)
        self.state.pool.release(seq_id)
        self.lengths.pop(seq_id, None)

    # -- the step ----------------------------------------------------------------------------------------------------
    def execute(self, entries: Sequence[dict], hidden_trace: Optional[list] = None) -> Optional[torch.Tensor]:
        """entries: dict(seq_id, tokens, want) -- the next tokens of live sequences.  Runs them as ONE batch from the cache and state
        earlier steps left; returns f32 logits [sum(len(want)), vocab] on the device in entry order (None if nothing is wanted)."""
        if not entries:
            return None
        rows = []
        for e in entries:
            sid, toks = e["seq_id"], e["tokens"]
            if sid not in self.lengths:
                raise BackendError(f"sequence {sid} was not admitted")
            start = self.lengths[sid]
            table = self.blocks.grow_to(sid, start + len(toks))
            rows.append(dict(tokens=toks, start=start, block_table=table, state_slot=self.state.pool.slot_of(sid), want=e.get("want", ())))
        prep = prepare_step(rows, self.block_size)
        if (self.decode_graphs and hidden_trace is None and all(len(e["tokens"]) == 1 and list(e.get("want", ())) == [0] for e in entries)
                and prep["block_tables"].shape[1] <= self.graph_width):
            if self.model.ensure_positions(int(prep["max_position"]) + 1):
                self._graphs.clear()             # captured steps point at the old tables
            g = self._graphs.get(len(entries))
            if g is None:
                g = self._graphs[len(entries)] = _DecodeGraph(self, len(entries), self.graph_width)
            logits = g.replay(prep)
        else:
            batch = StepBatch.from_host(prep, self.model.device)
            logits = self.model.forward(batch, self.cache.gpu_cache if self.cache else [], self.state.tensors, hidden_trace)
        for e in entries:
            self.lengths[e["seq_id"]] += len(e["tokens"])
        return logits


@dataclass
class Request:
    id: int
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    computed: int = 0                  # tokens already run through the model
    finished: bool = False

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output


class Scheduler:
    """FCFS continuous batching with chunked prefill.  A request is admitted when a state slot is free and the blocks for its prompt plus
    its ``max_tokens`` fit beside what the running requests have reserved, so a running request never has to be preempted."""

    def __init__(self, runner: ModelRunner, max_batch_tokens: int = 2048, max_num_seqs: int = 4, prefill_chunk: int = 512):
        self.runner, self.max_batch_tokens, self.max_num_seqs, self.prefill_chunk = runner, max_batch_tokens, max_num_seqs, prefill_chunk
        self.waiting: "deque[Request]" = deque()
        self.running: List[Request] = []

    def _blocks_for(self, r: Request) -> int:
        return -(-(len(r.prompt) + r.params.max_tokens) // self.runner.block_size)

    def _reserved(self) -> int:
        held = lambda r: len(self.runner.blocks.tables.get(r.id, ()))
        return sum(max(0, self._blocks_for(r) - held(r)) for r in self.running)

    def add(self, r: Request) -> None:
        if self._blocks_for(r) > self.runner.blocks.num_gpu_blocks:
            raise BackendError(f"request {r.id} needs {self._blocks_for(r)} blocks, the pool has {self.runner.blocks.num_gpu_blocks}")
        self.waiting.append(r)

    def schedule(self) -> List[dict]:
        """-> entries for ModelRunner.execute (each also carries its Request under 'request')"""
        while self.waiting and len(self.running) < self.max_num_seqs:
            r = self.waiting[0]
            if self.runner.state.pool.num_free() == 0 or self._blocks_for(r) > self.runner.blocks.num_free_gpu_blocks() - self._reserved():
                break
            self.waiting.popleft()
            self.runner.admit(r.id)
            self.running.append(r)
        budget, entries = self.max_batch_tokens, []
        for r in self.running:                       # decodes first: one token each
            if r.computed >= len(r.prompt) and budget > 0:
                entries.append(dict(seq_id=r.id, tokens=[r.tokens[-1]], want=[0], request=r))
                budget -= 1
        for r in self.running:                       # then prompt portions
            if r.computed < len(r.prompt) and budget > 0:
                n = min(len(r.prompt) - r.computed, self.prefill_chunk, budget)
                toks = r.prompt[r.computed:r.computed + n]
                last = r.computed + n == len(r.prompt)
                entries.append(dict(seq_id=r.id, tokens=toks, want=[n - 1] if last else [], request=r))
                budget -= n
        return entries

    def finish(self, r: Request) -> None:
        r.finished = True
        self.running.remove(r)
        self.runner.release(r.id)


class LLMEngine:
    def __init__(self, model, num_blocks: int = 256, max_num_seqs: int = 4, block_size: int = 64, max_batch_tokens: int = 2048,
                 prefill_chunk: int = 512, decode_graphs: bool = False, max_blocks_per_seq: int = 0):
        self.model = model
        self.runner = ModelRunner(model, num_blocks, max_num_seqs, block_size, decode_graphs=decode_graphs, max_blocks_per_seq=max_blocks_per_seq)
        self.scheduler = Scheduler(self.runner, max_batch_tokens, max_num_seqs, prefill_chunk)
        self.sampler = Sampler()
        self._next_id = 0
        self.steps = 0

    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, max_model_len: int = 4096, **kw) -> "LLMEngine":
        from .registry import load_model
        block_size = kw.get("block_size", 64)
        return cls(load_model(path, dtype=dtype, block_size=block_size, max_pos=max_model_len), **kw)

    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        if len(prompt) == 0:
            raise BackendError("empty prompt")
        r = Request(self._next_id, [int(t) for t in prompt], params or SamplingParams())
        self._next_id += 1
        self.scheduler.add(r)
        return r

    def has_work(self) -> bool:
        return bool(self.scheduler.waiting or self.scheduler.running)

    def step(self) -> List[Request]:
        """one scheduled batch through the model; returns the requests that finished in it"""
        entries = self.scheduler.schedule()
        if not entries:
            if self.scheduler.waiting:
                raise BackendError("scheduler stalled: a waiting request cannot be admitted and nothing is running")
            return []
        logits = self.runner.execute(entries)
        self.steps += 1
        done = []
        sampled = [e for e in entries if e["want"]]
        for e in entries:
            e["request"].computed += len(e["tokens"])
        if sampled:
            toks = self.sampler.sample(logits, [e["request"].params for e in sampled], [e["request"].id for e in sampled])
            for e, t in zip(sampled, toks):
                r = e["request"]
                r.output.append(t)
                if len(r.output) >= r.params.max_tokens or t in r.params.stop_token_ids:
                    self.scheduler.finish(r)
                    self.sampler.forget(r.id)
                    done.append(r)
        return done

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[List[int]]:
        ps = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        reqs = [self.add_request(p, q) for p, q in zip(prompts, ps)]
        while self.has_work():
            self.step()
        return [r.output for r in reqs]
