"""Ways of cutting the same requests into steps, shared by the replay tests.

A trace is a list of steps; a step is ``{"step": n, "entries": [{"id",
"tokens", "want"}], "end": [...]}``, the format ``bin/trace_run`` reads. The
expected logits of every wanted place are the plain implementation's logits of
the whole sequence at that position."""
import numpy as np


def whole(requests):
    """Each request alone, all its tokens in one step, every position wanted."""
    return [{"step": n, "entries": [{"id": name, "tokens": ids, "want": list(range(len(ids)))}],
             "end": [name]} for n, (name, ids) in enumerate(requests.items())]


def tail_by_one(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for name, ids in requests.items():
        head = max(len(ids) - tail, 1)
        steps.append({"entries": [{"id": name, "tokens": ids[:head], "want": [head - 1]}], "end": []})
        for i in range(head, len(ids)):
            steps.append({"entries": [{"id": name, "tokens": [ids[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [name]
    for n, step in enumerate(steps):
        step["step"] = n
    return steps


def ragged(requests, sizes=(7, 16, 2, 31, 2, 5, 64, 3, 17, 2, 1, 33)):
    """Portions of changing size, down to two tokens (and one)."""
    steps = []
    for name, ids in requests.items():
        cursor, turn = 0, 0
        while cursor < len(ids):
            size = min(sizes[turn % len(sizes)], len(ids) - cursor)
            steps.append({"entries": [{"id": name, "tokens": ids[cursor:cursor + size],
                                       "want": list(range(size))}], "end": []})
            cursor += size
            turn += 1
        steps[-1]["end"] = [name]
    for n, step in enumerate(steps):
        step["step"] = n
    return steps


def mixed(requests, seed, max_live=4, decode_tail=12):
    """Up to ``max_live`` requests live at a time: portions of some prompts
    beside single decoded tokens of others; a request may sit a step out; ended
    requests make room for the next. Returns the steps and the most tokens
    live requests hold at any time (each rounded up to 64)."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live = {}   # name -> [ids, cursor]
    steps, peak = [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            name, ids = waiting.pop(0)
            live[name] = [ids, 0]
        entries, ended = [], []
        for name, state in list(live.items()):
            ids, cursor = state
            if len(live) > 1 and rng.random() < 0.2:
                continue   # left out of this step
            left = len(ids) - cursor
            if left <= decode_tail:
                size = 1
            else:
                size = int(min(left - decode_tail, rng.choice([2, 3, 5, 8, 13, 16, 17, 29, 40])))
            entries.append({"id": name, "tokens": ids[cursor:cursor + size], "want": [size - 1] if size > 1 else [0]})
            state[1] += size
            if state[1] == len(ids):
                ended.append(name)
        held = sum(-(-state[1] // 64) * 64 for state in live.values())
        peak = max(peak, held)
        for name in ended:
            del live[name]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps, peak


def expected_rows(step, offsets, reference):
    """Rows of the plain logits for a step's wanted places. ``offsets[name]``
    is the position of the entry's first token."""
    rows = []
    for entry in step["entries"]:
        for index in entry["want"]:
            rows.append(reference[entry["id"]][offsets[entry["id"]] + index])
    return np.stack(rows) if rows else None


def replay(engine, steps, reference, StepEntry):
    """Feeds ``steps`` through ``engine.step``; returns the largest absolute
    difference from ``reference`` and the logits by (request, position)."""
    offsets, worst, seen = {}, 0.0, {}
    for step in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]]
        for e in step["entries"]:
            offsets.setdefault(e["id"], 0)
        logits = engine.step(entries)
        want = expected_rows(step, offsets, reference)
        if want is not None:
            got = logits.cpu().double().numpy()
            assert got.shape == want.shape
            worst = max(worst, float(np.abs(got - want).max()))
            row = 0
            for e in step["entries"]:
                for index in e["want"]:
                    seen[(e["id"], offsets[e["id"]] + index)] = got[row]
                    row += 1
        for e in step["entries"]:
            offsets[e["id"]] += len(e["tokens"])
        for name in step["end"]:
            engine.release(name)
            del offsets[name]
    engine.check()
    return worst, seen
