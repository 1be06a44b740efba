"""The slot scheduler of the serve surface: a host-side mirror of crates/ksearch_cli/src/scheduler.rs:78-353 over
`GemmaCudaModel`.

Same policy as the reference: requests wait in a queue and are admitted while slots are free (`admit`,
scheduler.rs:135-161); every tick runs a decode round over the requests in their decode phase, then a prefill round
that walks the prefilling requests round-robin under a token budget — small chunks while anything decodes, the
whole budget otherwise (scheduler.rs:233-304) — then frees the slots of finished requests.  A request finishes with
"length" (max_tokens, or the slot's context is full), "stop" (an end-of-sequence id, a stop string, or the same token
24 times in a row), "cancelled" (its sink refused a token) or "error".

One deliberate difference: the reference decodes its active requests one after the other (one `decode_token_sampled`
each, scheduler.rs:163-231); here the requests of a decode round that sit in neighbouring slots advance in ONE
model step (the backend's multi-slot path).  Greedy requests (temperature < 1e-6) take the device arg-max; the others
read their logits back and are sampled on the host with the reference's sampler (sample.rs:9-81)."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional

from .sample import sample_softcap_min_p

EOS_IDS = (1, 106)                                        # scheduler.rs:14
BUILTIN_STOPS = ("<turn|>", "<|turn>", "<tool_call|>")    # scheduler.rs:15
REPEAT_LIMIT = 24                                         # scheduler.rs:207


@dataclass
class InferenceRequest:                                   # scheduler.rs:28-36
    prompt_ids: list
    max_tokens: int = 64
    stop: list = field(default_factory=list)
    temperature: float = 0.0
    min_p: float = 0.05
    seed: int = 1
    on_event: Optional[Callable] = None                   # called with ("token", id) / ("done", reason, n_prompt, n_completion) / ("error", text); return False to cancel
    events: list = field(default_factory=list)            # the same events, kept when there is no callback

    def emit(self, *ev) -> bool:
        self.events.append(ev)
        return True if self.on_event is None else self.on_event(*ev) is not False


@dataclass
class SchedulerConfig:                                    # scheduler.rs:61-76
    slots: int = 4
    prefill_chunk: int = 128
    prefill_tokens_per_tick: int = 2048


@dataclass
class _Active:                                            # scheduler.rs:43-59
    req: InferenceRequest
    slot: int
    stop: list
    max_tokens: int
    rng: int
    cursor: int = 0               # prefill phase: prompt tokens already in the cache
    last_token: Optional[int] = None   # decode phase: the next input token (None while prefilling)
    generated: list = field(default_factory=list)
    text: str = ""
    finished: bool = False


class Scheduler:
    """`model`: slot_alloc / slot_free / slot_reset / seq_len / prefill / decode_token / forward / read_debug and a
    `cfg` with max_seq, vocab and softcap (GemmaCudaModel, or a stand-in with the same methods).
    `detokenize`: optional id -> text piece, for stop strings (the reference uses the model's vocabulary)."""

    def __init__(self, model, cfg: SchedulerConfig | None = None, detokenize: Optional[Callable] = None):
        self.model, self.cfg, self.detok = model, cfg or SchedulerConfig(), detokenize
        self.waiting: deque = deque()
        self.active: list = []
        self._prefill_next = 0

    def submit(self, req: InferenceRequest):
        self.waiting.append(req)

    def idle(self) -> bool:
        return not self.waiting and not self.active

    # ---- one pass of the reference's loop body (scheduler.rs:97-131)
    def tick(self):
        while len(self.active) < self.cfg.slots and self.waiting:
            req = self.waiting.popleft()
            if not req.prompt_ids:
                req.emit("error", "empty prompt")
                continue
            try:
                self.active.append(self._admit(req))
            except Exception as e:   # KvPool full and the like
                req.emit("error", f"admit failed: {e}")
        if not self.active:
            return
        self._decode_round()
        self._prefill_round()
        for a in self.active:
            if a.finished:
                self.model.slot_free(a.slot)
        self.active = [a for a in self.active if not a.finished]

    def run(self, max_ticks: int = 1 << 20):
        for _ in range(max_ticks):
            if self.idle():
                return
            self.tick()
        raise RuntimeError("scheduler did not drain")

    def _admit(self, req: InferenceRequest) -> _Active:
        slot = self.model.slot_alloc()
        self.model.slot_reset(slot)
        stop = list(req.stop) + [s for s in BUILTIN_STOPS if s not in req.stop]
        return _Active(req, slot, stop, max(int(req.max_tokens), 1), (int(req.seed) | 1) & 0xFFFFFFFF)

    def _finish(self, a: _Active, reason: str):            # scheduler.rs:330-353
        if a.finished:
            return
        a.finished = True
        if reason != "error":
            a.req.emit("done", reason, len(a.req.prompt_ids), len(a.generated))

    # ---- decode round (scheduler.rs:163-231), neighbouring slots in one model step
    def _decode_round(self):
        ready = []
        for a in self.active:
            if a.finished or a.last_token is None:
                continue
            if len(a.generated) >= a.max_tokens or self.model.seq_len(a.slot) >= self.model.cfg.max_seq:
                self._finish(a, "length")
                continue
            ready.append(a)
        ready.sort(key=lambda a: a.slot)
        i = 0
        while i < len(ready):
            j = i + 1
            while j < len(ready) and ready[j].slot == ready[j - 1].slot + 1:
                j += 1
            self._decode_run(ready[i:j])
            i = j

    def _decode_run(self, run):
        first, ids = run[0].slot, [a.last_token for a in run]
        for a in run:
            a.rng = (a.rng + 0x9E3779B9) & 0xFFFFFFFF
        try:
            if all(a.req.temperature < 1e-6 for a in run):
                nxt = self.model.decode_token(ids, first)          # device arg-max after the softcap
            else:
                self.model.forward(first, len(run), ids, True)
                self.model.ctx.synchronize()
                nxt = [sample_softcap_min_p(self.model.read_debug(1, a.slot), self.model.cfg.softcap, a.req.temperature,
                                            a.req.min_p, a.rng) for a in run]
        except Exception as e:
            for a in run:
                a.req.emit("error", str(e))
                self._finish(a, "error")
            return
        for a, tok in zip(run, nxt):
            self._take_token(a, int(tok))

    def _take_token(self, a: _Active, tok: int):
        a.last_token = tok
        if tok in EOS_IDS:
            return self._finish(a, "stop")
        if self.detok is not None:
            a.text += self.detok(tok)
            hit = next((s for s in a.stop if s and s in a.text), None)
            if hit is not None:
                a.text = a.text[:a.text.find(hit)]
                return self._finish(a, "stop")
        a.generated.append(tok)
        if len(a.generated) >= REPEAT_LIMIT and all(t == tok for t in a.generated[-REPEAT_LIMIT:]):
            return self._finish(a, "stop")
        if not a.req.emit("token", tok):
            return self._finish(a, "cancelled")
        if len(a.generated) >= a.max_tokens:
            self._finish(a, "length")

    # ---- prefill round (scheduler.rs:233-304)
    def _prefill_round(self):
        n = len(self.active)
        if n == 0 or not any(a.last_token is None and not a.finished for a in self.active):
            return
        decoding = any(not a.finished and a.last_token is not None for a in self.active)
        budget = max(self.cfg.prefill_tokens_per_tick, self.cfg.prefill_chunk)
        idx = self._prefill_next % n
        for _ in range(n):
            if budget == 0:
                break
            a = self.active[idx]
            idx = (idx + 1) % n
            if a.finished or a.last_token is not None:
                continue
            end = max(len(a.req.prompt_ids) - 1, 0)   # the last prompt token is the first decode input
            if a.cursor >= end:
                a.last_token = int(a.req.prompt_ids[-1])
                continue
            cap = self.cfg.prefill_chunk if decoding else budget
            take = min(budget, cap, end - a.cursor)
            try:
                self.model.prefill(a.slot, a.req.prompt_ids[a.cursor:a.cursor + take])
            except Exception as e:
                a.req.emit("error", str(e))
                self._finish(a, "error")
                continue
            budget -= take
            a.cursor += take
            if a.cursor >= end:
                a.last_token = int(a.req.prompt_ids[-1])
        self._prefill_next = idx
