"""The serving loop over any registered model: requests, state slots, portions, sampling.

A model plugs in through three members: `state_specs()` (what a sequence carries between steps), `vocab`, and
`forward_portion(tokens, ctx, want)` (run the next tokens of one sequence from the state earlier steps left,
return f32 logits at the wanted places).  The engine owns the `SequenceStatePool`, maps request ids to slots,
and offers two ways in:

  * `step(entries, end)`: the caller decides which tokens each request gets in this step (a replayed trace,
    an external scheduler);
  * `add_request()` + `run()` / `generate()`: the engine's own scheduler: waiting requests are admitted while
    slots and the token budget allow, prompts are fed in portions of at most `prefill_chunk` tokens, live
    requests take turns (one portion or one decoded token per turn), finished ones give their slot back.

Single-token steps are replayed as a CUDA graph once warm (slot and position are read on the device)."""
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from .mixers import StepContext
from .state import PoolFull, SequenceStatePool


@dataclass
class Request:
    request_id: Hashable
    prompt: List[int]
    max_new_tokens: int
    temperature: float = 0.0
    top_k: Optional[int] = None
    eos_id: Optional[int] = None
    fed: int = 0                                     # prompt tokens already run
    output: List[int] = field(default_factory=list)
    done: bool = False


class Engine:
    #: replay single-token steps as a CUDA graph after this many eager ones (0 = never)
    graph_after: int = 2

    def __init__(self, model, *, n_slots: int = 4, max_tokens: int = 0, prefill_chunk: int = 512, device: Optional[torch.device] = None) -> None:
        self.model = model
        self.device = torch.device(device) if device is not None else model.device
        self.pool = SequenceStatePool(model.state_specs(), n_slots, self.device, max_tokens=max_tokens)
        self.prefill_chunk = int(prefill_chunk)
        self.waiting: deque = deque()
        self.live: "OrderedDict[Hashable, Request]" = OrderedDict()
        self.finished: Dict[Hashable, Request] = {}
        self._meta = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._tok1 = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._want0 = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._graph = None
        self._graph_out: Optional[torch.Tensor] = None
        self._single_calls = 0
        self.steps = 0

    # ------------------------------------------------------------------ one portion of one request
    def _run(self, request_id: Hashable, tokens: Sequence[int], want: Optional[Sequence[int]]) -> torch.Tensor:
        """Feed `tokens` to the request's sequence; f32 logits [len(want), vocab] (want None: the last token)."""
        T = len(tokens)
        if T == 0:
            return torch.empty((0, self.model.vocab), dtype=torch.float32, device=self.device)
        if not self.pool.has(request_id):
            self.pool.acquire(request_id)
        self.pool.reserve(request_id, T)
        slot, pos0 = self.pool.slot(request_id), self.pool.position(request_id)
        cap = getattr(self.model, "max_positions", 0)          # models that cache every position say how many fit a slot
        if cap and pos0 + T > cap:
            raise PoolFull(f"request {request_id!r} would reach position {pos0 + T}, a slot holds {cap}")
        self._meta.copy_(torch.tensor([slot, pos0], dtype=torch.int32))
        want = [T - 1] if want is None else list(want)
        if any(w < 0 or w >= T for w in want):
            raise IndexError(f"wanted places {want} outside a portion of {T} tokens")
        graphable = T == 1 and want == [0] and self.graph_after > 0 and getattr(self.model, "graph_safe", True)
        if graphable:
            self._tok1.copy_(torch.tensor(list(tokens), dtype=torch.int64))
            out = self._single_token()
        else:
            tok = torch.tensor(list(tokens), dtype=torch.int64).to(self.device)
            w = torch.tensor(want, dtype=torch.int32).to(self.device) if want else None
            ctx = StepContext(T, self._meta, self.pool.tensors, self.model.dtype, pos_hint=pos0, slot_hint=slot)
            out = self.model.forward_portion(tok, ctx, w) if want else self._no_logits(tok, ctx)
        self.pool.advance(request_id, T)
        self.steps += 1
        return out

    def _no_logits(self, tok: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        self.model.forward_portion(tok, ctx, torch.empty(0, dtype=torch.int32, device=self.device))
        return torch.empty((0, self.model.vocab), dtype=torch.float32, device=self.device)

    def _single_token(self) -> torch.Tensor:
        if self._graph is not None:
            self._graph.replay()
            return self._graph_out.clone()
        self._single_calls += 1
        if self._single_calls > self.graph_after:
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                ctx = StepContext(1, self._meta, self.pool.tensors, self.model.dtype)    # inside: it records the capturing stream
                self._graph_out = self.model.forward_portion(self._tok1, ctx, self._want0)
            self._graph = g
            g.replay()            # capture does not run the kernels: this replay is the step itself
            return self._graph_out.clone()
        ctx = StepContext(1, self._meta, self.pool.tensors, self.model.dtype)
        return self.model.forward_portion(self._tok1, ctx, self._want0)

    # ------------------------------------------------------------------ caller-scheduled steps
    def step(self, entries: Sequence[dict], end: Sequence[Hashable] = ()) -> List[torch.Tensor]:
        """entries: [{'id', 'tokens', 'want'}]: each request's next tokens and the places among them whose logits
        are wanted.  Returns one [len(want), vocab] f32 tensor per entry.  Requests in `end` give their state back
        after the step."""
        outs = [self._run(e["id"], e["tokens"], e.get("want", [])) for e in entries]
        for rid in end:
            if self.pool.has(rid):
                self.pool.release(rid)
        return outs

    # ------------------------------------------------------------------ the engine's own scheduler
    def add_request(self, request_id: Hashable, prompt: Sequence[int], max_new_tokens: int, *, temperature: float = 0.0,
                    top_k: Optional[int] = None, eos_id: Optional[int] = None) -> None:
        if not prompt:
            raise ValueError("empty prompt")
        if request_id in self.live or request_id in self.finished or any(r.request_id == request_id for r in self.waiting):
            raise KeyError(f"request id {request_id!r} is in use")
        self.waiting.append(Request(request_id, list(prompt), int(max_new_tokens), float(temperature), top_k, eos_id))

    def _admit(self) -> None:
        while self.waiting and self.pool.free_slots() > 0:
            r = self.waiting[0]
            need = len(r.prompt) + r.max_new_tokens
            if self.pool.max_tokens:
                booked = sum(len(q.prompt) + q.max_new_tokens for q in self.live.values())
                if booked + need > self.pool.max_tokens:
                    if not self.live:
                        raise PoolFull(f"request {r.request_id!r} needs {need} tokens, the budget is {self.pool.max_tokens}")
                    break
            self.waiting.popleft()
            self.pool.acquire(r.request_id)
            self.live[r.request_id] = r

    def _sample(self, logits: torch.Tensor, r: Request) -> int:
        if r.temperature <= 0.0:
            return int(torch.argmax(logits))
        from .generate import sample_token     # the package's fused temperature / top-k / draw kernel (bf16 logits)

        return int(sample_token(logits.to(torch.bfloat16), r.temperature, r.top_k))

    def _turn(self, r: Request) -> None:
        if r.fed < len(r.prompt):
            part = r.prompt[r.fed: r.fed + self.prefill_chunk]
            r.fed += len(part)
            last = r.fed == len(r.prompt)
            out = self._run(r.request_id, part, [len(part) - 1] if last else [])
            if not last:
                return
        else:
            out = self._run(r.request_id, [r.output[-1]], [0])
        if r.max_new_tokens <= 0:
            r.done = True
            return
        tok = self._sample(out[0], r)
        r.output.append(tok)
        if len(r.output) >= r.max_new_tokens or (r.eos_id is not None and tok == r.eos_id):
            r.done = True

    def run(self) -> Dict[Hashable, List[int]]:
        """Serve until every request is finished; request id -> generated tokens (the EOS token included)."""
        while self.waiting or self.live:
            self._admit()
            for rid in list(self.live):
                r = self.live[rid]
                self._turn(r)
                if r.done:
                    del self.live[rid]
                    self.pool.release(rid)
                    self.finished[rid] = r
        out = {rid: r.output for rid, r in self.finished.items()}
        self.finished = {}
        return out

    def generate(self, prompt: Sequence[int], max_new_tokens: int, **kw) -> List[int]:
        """One request through the scheduler: prompt + generated tokens."""
        rid = ("generate", self.steps, len(self.finished))
        self.add_request(rid, prompt, max_new_tokens, **kw)
        return list(prompt) + self.run()[rid]
