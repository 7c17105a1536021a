"""The scheduler's decisions with a fake step over the real cache manager (no
GPU), after the reference's FakeDecoder tests
(crates/app/cli/src/engine_loop.rs:1423-1816, :1923-2905): the fake's next
token depends only on the request's own tokens, so batching, portions and
preemption must not change any output."""
import pytest

from metallix_b200.csrc import build

VOCAB = 97


@pytest.fixture(scope="module")
def host():
    return build.host()


def next_token(context):
    return sum((i + 1) * t for i, t in enumerate(context)) % VOCAB


class Driver:
    """Runs plans against the real manager; records every plan."""

    def __init__(self, host, pages=64, page_tokens=4, max_requests=8, **limits):
        self.host = host
        self.manager = host.CacheManager([host.GroupConfig(page_tokens, 0, pages)], max_requests)
        self.scheduler = host.Scheduler(self.manager, host.Limits(**limits))
        self.plans = []

    def add(self, prompt, max_new_tokens, stop=(), ignore_eos=False):
        return self.scheduler.add(list(prompt), max_new_tokens, list(stop), ignore_eos)

    def step(self):
        plan = self.scheduler.plan()
        self.plans.append(plan)
        tokens = []
        for entry in plan.entries:
            assert self.manager.computed(entry.id) == entry.start
            self.manager.reserve(entry.id, len(entry.tokens))
            self.manager.commit(entry.id, len(entry.tokens))
            info = self.scheduler.request(entry.id)
            context = list(info.prompt) + list(info.output)
            assert context[entry.start:entry.start + len(entry.tokens)] == list(entry.tokens)
            if entry.wants_token:
                assert entry.start + len(entry.tokens) == len(context)
                assert entry.generated_position == len(info.output)
                tokens.append(next_token(context))
        self.manager.check_invariants()
        return plan, self.scheduler.update(plan, tokens)

    def run(self, limit=10_000):
        for _ in range(limit):
            if self.scheduler.idle():
                return
            self.step()
        raise AssertionError("the scheduler did not finish")

    def output(self, rid):
        return list(self.scheduler.request(rid).output)


def serial(prompt, count, stop=()):
    context, out = list(prompt), []
    for _ in range(count):
        token = next_token(context)
        out.append(token)
        context.append(token)
        if token in stop:
            break
    return out


PROMPTS = [[(7 * i + j * j) % VOCAB for j in range(n)] for i, n in enumerate([5, 17, 31, 1, 9, 40, 63, 12])]


def test_batched_equals_serial(host):
    d = Driver(host, pages=128, max_num_seqs=4, max_tokens_per_step=64)
    ids = [d.add(p, 16) for p in PROMPTS]
    d.run()
    for rid, prompt in zip(ids, PROMPTS):
        assert d.output(rid) == serial(prompt, 16)
        assert d.scheduler.request(rid).finish_reason == "length"
    assert d.manager.free_pages(0) == 128 and d.manager.live_requests() == 0
    assert max(len(p.entries) for p in d.plans) == 4   # never more than max_num_seqs together


def test_decoded_tokens_first_then_portions_under_the_budget(host):
    d = Driver(host, pages=128, max_num_seqs=4, max_tokens_per_step=24, prefill_chunk=16)
    a = d.add(PROMPTS[0], 8)
    d.step()                                # a's whole prompt (5 tokens)
    b = d.add(PROMPTS[6], 4)                # 63 tokens: portions of 16
    plan, _ = d.step()
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(a, 1), (b, 16)]
    assert plan.decode_tokens == 1 and plan.prefill_tokens == 16
    c = d.add(PROMPTS[2], 4)                # 31 tokens
    plan, _ = d.step()
    # budget 24: one decoded token, b's next 16, then 7 left for c
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(a, 1), (b, 16), (c, 7)]
    assert [e.wants_token for e in plan.entries] == [True, False, False]
    sizes = []
    while not d.scheduler.idle():
        plan, _ = d.step()
        assert sum(len(e.tokens) for e in plan.entries) <= 24
        sizes += [len(e.tokens) for e in plan.entries if e.id == b and len(e.tokens) > 1]
    assert sizes[:2] == [16, 15]            # 63 = 16 + 16 + 16 + 15
    for rid, prompt, n in ((a, PROMPTS[0], 8), (b, PROMPTS[6], 4), (c, PROMPTS[2], 4)):
        assert d.output(rid) == serial(prompt, n)


def test_tiny_pool_preempts_and_outputs_stay(host):
    # 14 pages of 4: the three requests cannot all grow to the end.
    d = Driver(host, pages=14, max_num_seqs=3, max_tokens_per_step=64)
    ids = [d.add(p, 20) for p in PROMPTS[:3]]
    d.run()
    preempted = [rid for plan in d.plans for rid in plan.preempted]
    assert preempted, "the pool was meant to run out"
    for rid, prompt in zip(ids, PROMPTS[:3]):
        assert d.output(rid) == serial(prompt, 20)
    assert sum(d.scheduler.request(rid).preemptions for rid in ids) == len(preempted)
    assert d.manager.free_pages(0) == 14


def test_the_victim_is_the_last_admitted_and_returns_to_the_front(host):
    d = Driver(host, pages=7, page_tokens=4, max_num_seqs=2, max_tokens_per_step=64)
    a = d.add([1] * 12, 12)   # 3 pages
    b = d.add([2] * 11, 12)   # 3 pages; admission needs 3 + 1 headroom <= 4 free
    c = d.add([3] * 4, 4)
    d.step()
    assert d.scheduler.running() == [a, b] and d.scheduler.waiting() == [c]
    victims = []
    for _ in range(6):
        plan, _ = d.step()
        victims += plan.preempted
        if victims:
            break
    assert victims == [b]                       # engine_loop.rs:1138-1167: the newest row
    assert d.scheduler.waiting()[0] == b        # in front of c, with everything it produced
    d.run()
    assert d.output(a) == serial([1] * 12, 12) and d.output(b) == serial([2] * 11, 12)
    assert d.output(c) == serial([3] * 4, 4)


def test_a_lone_request_that_outgrows_the_pool_fails(host):
    d = Driver(host, pages=3, max_num_seqs=2, max_tokens_per_step=64)
    rid = d.add([5] * 10, 30)
    d.run()
    info = d.scheduler.request(rid)
    assert info.failed and info.finish_reason == "the sequence outgrew the KV pool"
    assert len(info.output) == 3                 # 12 positions fit: 10 prompt + 2 decoded inputs
    assert d.manager.free_pages(0) == 3 and d.manager.live_requests() == 0


def test_a_prompt_larger_than_the_pool_fails_at_once(host):
    d = Driver(host, pages=3, max_num_seqs=2, max_tokens_per_step=64)
    big = d.add([5] * 13, 4)
    small = d.add([6] * 3, 2)
    d.run()
    assert d.scheduler.request(big).finish_reason == "the prompt does not fit the KV pool"
    assert d.output(small) == serial([6] * 3, 2)


def test_admission_keeps_headroom(host):
    d = Driver(host, pages=8, max_num_seqs=4, max_tokens_per_step=64)
    a = d.add([1] * 8, 8)     # 2 pages
    d.step()
    # a's next token claims a third page; 6 pages are free
    b = d.add([2] * 16, 4)    # 1 claimed + 4 pages + 1 headroom = 6 <= 6: admitted
    c = d.add([3] * 4, 4)     # 5 claimed + 1 page + 2 headroom > 6: waits
    plan, _ = d.step()
    assert [e.id for e in plan.entries] == [a, b]
    assert d.scheduler.waiting() == [c]
    d.run()
    assert d.output(c) == serial([3] * 4, 4)


def test_stop_ids_and_ignore_eos(host):
    prompt = PROMPTS[1]
    free_run = serial(prompt, 12)
    stop = free_run[4]
    d = Driver(host, max_num_seqs=2)
    a = d.add(prompt, 12, stop=[stop])
    b = d.add(prompt, 12, stop=[stop], ignore_eos=True)
    d.run()
    cut = free_run.index(stop) + 1
    assert d.output(a) == free_run[:cut] and d.scheduler.request(a).finish_reason == "eos"
    assert d.output(b) == free_run and d.scheduler.request(b).finish_reason == "length"


def test_cancel_frees_pages(host):
    d = Driver(host, pages=32, max_num_seqs=2, max_tokens_per_step=64)
    a = d.add(PROMPTS[2], 50)
    b = d.add(PROMPTS[1], 6)
    waiting = d.add(PROMPTS[0], 6)
    d.step()
    d.step()
    held = d.manager.free_pages(0)
    d.scheduler.cancel(a)
    d.scheduler.cancel(waiting)
    d.step()
    assert d.scheduler.request(a).finish_reason == "cancelled"
    assert d.scheduler.request(waiting).finish_reason == "cancelled"
    assert d.manager.free_pages(0) > held and not d.manager.has(a)
    d.run()
    assert d.output(b) == serial(PROMPTS[1], 6)
    assert d.manager.free_pages(0) == 32


def test_a_deadline_ends_a_request_wherever_it_is(host):
    """Deadlines on the caller's clock (engine_loop.rs:631-653, :932-943): a
    request whose deadline has passed leaves at the next plan, keeping what it
    generated and giving its pages back, whether it decodes, waits or is in its
    prompt; requests without a deadline go on."""
    d = Driver(host, pages=32, max_num_seqs=2, max_tokens_per_step=8)
    sampling = host.SamplingParams()
    decoding = d.scheduler.add(list(PROMPTS[1]), 50, [], False, sampling, 10.0)
    free = d.scheduler.add(list(PROMPTS[0]), 6, [], False, sampling)
    waiting = d.scheduler.add(list(PROMPTS[2]), 6, [], False, sampling, 10.0)

    def step(now):
        plan = d.scheduler.plan(now)
        tokens = []
        for entry in plan.entries:
            d.manager.reserve(entry.id, len(entry.tokens))
            d.manager.commit(entry.id, len(entry.tokens))
            info = d.scheduler.request(entry.id)
            if entry.wants_token:
                tokens.append(next_token(list(info.prompt) + list(info.output)))
        d.scheduler.update(plan, tokens)

    for now in (1.0, 2.0, 3.0, 9.9):
        step(now)
    assert d.scheduler.request(decoding).finish_reason == "" and d.scheduler.waiting() == [waiting]
    generated = len(d.scheduler.request(decoding).output)
    step(10.0)
    assert d.scheduler.request(decoding).finish_reason == "deadline"
    assert d.scheduler.request(waiting).finish_reason == "deadline"
    assert len(d.scheduler.request(decoding).output) == generated and not d.manager.has(decoding)
    while not d.scheduler.idle():
        step(11.0)
    assert d.output(free) == serial(PROMPTS[0], 6) and d.scheduler.request(free).finish_reason == "length"
    assert d.manager.free_pages(0) == 32
    # in its prompt: portions of 8 tokens, the deadline passes after the first
    long_prompt = d.scheduler.add([3] * 30, 4, [], False, sampling, 20.0)
    step(19.0)
    assert d.manager.has(long_prompt) and 0 < d.manager.computed(long_prompt) < 30
    step(20.5)
    assert d.scheduler.request(long_prompt).finish_reason == "deadline" and d.manager.free_pages(0) == 32


def test_failed_step_releases_its_requests(host):
    d = Driver(host, pages=32, max_num_seqs=2)
    a = d.add(PROMPTS[0], 4)
    plan = d.scheduler.plan()
    d.scheduler.fail_plan(plan, "step failed: injected")
    assert d.scheduler.request(a).failed and d.scheduler.idle()
    assert d.manager.free_pages(0) == 32 and d.manager.live_requests() == 0


def test_invalid_requests(host):
    d = Driver(host)
    with pytest.raises(ValueError):
        d.add([], 4)
    with pytest.raises(ValueError):
        d.add([1], 0)
    with pytest.raises(ValueError):
        host.Scheduler(d.manager, host.Limits(max_num_seqs=99))
