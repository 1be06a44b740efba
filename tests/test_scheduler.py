"""The slot scheduler (crates/ksearch_cli/src/scheduler.rs:78-353) against a stand-in model on the CPU: admission,
the prefill budget and its fairness rule, the finish reasons, and the grouping of neighbouring slots into one step."""
import pytest

from ksearch_b200.scheduler import EOS_IDS, InferenceRequest, Scheduler, SchedulerConfig


class _Cfg:
    def __init__(self, max_seq, vocab=1000, softcap=30.0):
        self.max_seq, self.vocab, self.softcap = max_seq, vocab, softcap


class FakeModel:
    """Slots with a length each; the next token is a fixed function of (input token, context length)."""

    def __init__(self, n_slots=4, max_seq=64, rule=None):
        self.cfg = _Cfg(max_seq)
        self.n_slots, self.used, self.len = n_slots, set(), {}
        self.rule = rule or (lambda tok, n: (tok * 7 + n) % 997 + 200)     # never an end-of-sequence id
        self.prefills, self.steps = [], []

    def slot_alloc(self):
        for s in range(self.n_slots):
            if s not in self.used:
                self.used.add(s)
                self.len[s] = 0
                return s
        raise RuntimeError("KvPool full")

    def slot_free(self, s):
        self.used.discard(s)

    def slot_reset(self, s):
        self.len[s] = 0

    def seq_len(self, s):
        return self.len[s]

    def prefill(self, s, toks):
        assert s in self.used and self.len[s] + len(toks) <= self.cfg.max_seq
        self.prefills.append((s, len(toks)))
        self.len[s] += len(toks)

    def decode_token(self, toks, first=0):
        self.steps.append((first, len(toks)))
        out = []
        for i, t in enumerate(toks):
            s = first + i
            assert s in self.used
            out.append(self.rule(t, self.len[s]))
            self.len[s] += 1
        return out


def _tokens(req):
    return [e[1] for e in req.events if e[0] == "token"]


def _done(req):
    d = [e for e in req.events if e[0] == "done"]
    return d[0][1:] if d else None


def test_requests_run_to_their_lengths_and_slots_are_reused():
    m = FakeModel(n_slots=2)
    s = Scheduler(m, SchedulerConfig(slots=2, prefill_chunk=4, prefill_tokens_per_tick=8))
    reqs = [InferenceRequest(list(range(300, 300 + n)), max_tokens=k) for n, k in ((5, 3), (1, 6), (9, 2), (2, 4))]
    for r in reqs:
        s.submit(r)
    s.run(200)
    for r, (n, k) in zip(reqs, ((5, 3), (1, 6), (9, 2), (2, 4))):
        assert _done(r) == ("length", n, k) and len(_tokens(r)) == k
    assert m.used == set() and s.idle()
    # each request's tokens follow the model's rule from its own history, whatever ran beside it
    r = reqs[0]
    tok, n, want = r.prompt_ids[-1], len(r.prompt_ids) - 1, []
    for _ in range(3):
        tok = m.rule(tok, n)
        want.append(tok)
        n += 1
    assert _tokens(r) == want
    assert any(n == 2 for _, n in m.steps)               # two neighbouring slots advanced in one step


def test_prefill_budget_and_fairness():
    m = FakeModel(n_slots=3, max_seq=4096)
    s = Scheduler(m, SchedulerConfig(slots=3, prefill_chunk=16, prefill_tokens_per_tick=100))
    long_a, long_b = InferenceRequest(list(range(200, 200 + 301)), max_tokens=2), InferenceRequest(list(range(200, 200 + 151)), max_tokens=2)
    s.submit(long_a)
    s.submit(long_b)
    s.tick()                                              # nothing decodes yet: the whole budget goes to prefill
    assert m.prefills == [(0, 100)]
    s.tick()
    assert m.prefills[1:] == [(1, 100)]                   # round-robin: the other request's turn
    s.submit(InferenceRequest([7, 8], max_tokens=50))    # a short prompt starts decoding after one tick
    s.tick()
    s.tick()
    before = len(m.prefills)
    s.tick()                                              # something decodes now: prefill in chunks of prefill_chunk
    assert all(n <= 16 for _, n in m.prefills[before:]) and sum(n for _, n in m.prefills[before:]) <= 100
    s.run(500)
    assert sum(n for sl, n in m.prefills if sl == 0) == 300 and _done(long_a) == ("length", 301, 2)


def test_finish_reasons():
    # end-of-sequence id
    m = FakeModel(rule=lambda tok, n: EOS_IDS[1] if n >= 3 else 500 + n)
    s = Scheduler(m, SchedulerConfig(slots=1))
    r = InferenceRequest([300, 301], max_tokens=50)
    s.submit(r)
    s.run(100)
    assert _done(r) == ("stop", 2, 2) and _tokens(r) == [501, 502]
    # the same token 24 times
    m = FakeModel(rule=lambda tok, n: 555)
    s = Scheduler(m, SchedulerConfig(slots=1))
    r = InferenceRequest([300], max_tokens=100)
    s.submit(r)
    s.run(200)
    assert _done(r) == ("stop", 1, 24) and len(_tokens(r)) == 23      # the 24th is counted but not sent
    # the slot's context is full
    m = FakeModel(max_seq=6)
    s = Scheduler(m, SchedulerConfig(slots=1))
    r = InferenceRequest([300, 301, 302], max_tokens=100)
    s.submit(r)
    s.run(100)
    assert _done(r)[0] == "length" and len(_tokens(r)) == 4          # positions 2..5, then the cache is full
    # a stop string through the detokenizer: the text is cut at the stop, the token is not sent
    m = FakeModel(rule=lambda tok, n: 600 + n)
    s = Scheduler(m, SchedulerConfig(slots=1), detokenize=lambda t: "<turn|>" if t == 603 else "ab")
    r = InferenceRequest([300, 301], max_tokens=50)
    s.submit(r)
    s.run(100)
    assert _done(r) == ("stop", 2, 2) and _tokens(r) == [601, 602]
    # the sink refuses a token
    m = FakeModel()
    s = Scheduler(m, SchedulerConfig(slots=1))
    seen = []
    r = InferenceRequest([300], max_tokens=50, on_event=lambda *ev: (seen.append(ev), len(seen) < 3)[1])
    s.submit(r)
    s.run(100)
    assert _done(r)[0] == "cancelled" and len(_tokens(r)) == 3
    # empty prompt, and a model error
    s = Scheduler(FakeModel(), SchedulerConfig(slots=1))
    r = InferenceRequest([])
    s.submit(r)
    s.run(10)
    assert r.events == [("error", "empty prompt")]

    class Broken(FakeModel):
        def decode_token(self, toks, first=0):
            raise RuntimeError("device said no")
    m = Broken()
    s = Scheduler(m, SchedulerConfig(slots=1))
    r = InferenceRequest([300, 301], max_tokens=5)
    s.submit(r)
    s.run(10)
    assert r.events == [("error", "device said no")] and m.used == set()


def test_more_requests_than_slots_wait_their_turn():
    m = FakeModel(n_slots=2)
    s = Scheduler(m, SchedulerConfig(slots=2))
    reqs = [InferenceRequest([300 + i], max_tokens=3) for i in range(5)]
    for r in reqs:
        s.submit(r)
    s.tick()
    assert len(s.active) == 2 and len(s.waiting) == 3
    s.run(100)
    assert all(_done(r) == ("length", 1, 3) for r in reqs)
    # the scheduler asks for a slot only while it has fewer than cfg.slots active, so a smaller pool reports the failure
    m = FakeModel(n_slots=1)
    s = Scheduler(m, SchedulerConfig(slots=2))
    a, b = InferenceRequest([300], max_tokens=2), InferenceRequest([301], max_tokens=2)
    s.submit(a)
    s.submit(b)
    s.run(50)
    assert _done(a) == ("length", 1, 2) and b.events[0][0] == "error" and "admit failed" in b.events[0][1]


def test_sampled_requests_read_logits_and_use_the_reference_sampler():
    """temperature > 0: the step runs with logits, each request's row goes through sample_softcap_min_p with the
    request's own rng state (seed | 1, advanced by 0x9E3779B9 per step, scheduler.rs:181-182)."""
    import numpy as np
    from ksearch_b200.sample import sample_softcap_min_p

    class LogitModel(FakeModel):
        class _Ctx:
            def synchronize(self):
                pass
        ctx = _Ctx()

        def forward(self, first, n, toks, want_logits):
            assert want_logits
            self.steps.append((first, n))
            self.rows = {}
            for i, t in enumerate(toks):
                s = first + i
                rng = np.random.default_rng(1000 * t + self.len[s])
                self.rows[s] = (rng.standard_normal(self.cfg.vocab) * 3).astype(np.float32)
                self.rows[s][[1, 106]] = -50.0            # never an end-of-sequence id
                self.len[s] += 1

        def read_debug(self, which, slot):
            assert which == 1
            return self.rows[slot]

    m = LogitModel(n_slots=2)
    s = Scheduler(m, SchedulerConfig(slots=2))
    a = InferenceRequest([300, 301], max_tokens=4, temperature=0.9, min_p=0.05, seed=10)
    b = InferenceRequest([400], max_tokens=4, temperature=0.0)          # greedy beside it: the mixed step samples both on the host
    s.submit(a)
    s.submit(b)
    s.run(50)
    assert _done(a) == ("length", 2, 4) and _done(b) == ("length", 1, 4)
    # replay request a alone with the documented rng sequence
    m2 = LogitModel(n_slots=1)
    m2.slot_alloc()
    m2.prefill(0, [300])
    tok, rng, want = 301, (10 | 1), []
    for _ in range(4):
        rng = (rng + 0x9E3779B9) & 0xFFFFFFFF
        m2.forward(0, 1, [tok], True)
        tok = sample_softcap_min_p(m2.read_debug(1, 0), 30.0, 0.9, 0.05, rng)
        want.append(tok)
    assert _tokens(a) == want
    # the greedy request got the arg-max of its rows
    m3 = LogitModel(n_slots=2)
    m3.slot_alloc(); m3.slot_alloc()
    tok, got = 400, _tokens(b)
    for step in range(4):
        m3.forward(1, 1, [tok], True)
        tok = int(np.argmax(30.0 * np.tanh(m3.read_debug(1, 1) / 30.0)))
        assert got[step] == tok
