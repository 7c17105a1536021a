"""Generation through the scheduler: the Python entry point.

``Generator`` owns a C++ ``Scheduler`` over the engine's cache manager. Each
iteration asks the scheduler for a plan (decoded tokens of running requests
first, then portions of prompts under the token budget, then admissions), runs
it as ONE engine step, picks a token on the device for every entry that reached
the end of what it knows, and hands the tokens back; the scheduler finishes and
frees. The loop is the reference's ``Engine::step``
(crates/app/cli/src/engine_loop.rs:618-677); the receipt's field names are
those of ``mx gen`` (crates/app/cli/src/qwen_forward.rs:1021-1050).
"""
from __future__ import annotations

import contextlib
import json
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..csrc import build
from ..sampling import SamplingParams, pick
from .engine import Engine, StepEntry


@dataclass
class GenerationResult:
    input_ids: List[int]
    generated_ids: List[int]
    finish_reason: str          # "eos", "length", "cancelled", or an error text
    failed: bool = False
    preemptions: int = 0
    cached_tokens: int = 0      # positions the request held when it finished
    prefill_ms: float = 0.0     # from admission to its first token
    decode_ms: List[float] = field(default_factory=list)  # per later token


@dataclass
class GenerationStats:
    steps: int = 0
    decode_tokens: int = 0
    prefill_tokens: int = 0
    preemptions: int = 0
    ahead_kept: int = 0       # steps launched before their tokens reached the host, and kept
    ahead_dropped: int = 0    # ... and dropped because the scheduler decided otherwise
    step_ms: List[float] = field(default_factory=list)


class _DeviceSpan:
    def __init__(self, store: dict, key: int):
        self.store, self.key = store, key

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def __exit__(self, *exc):
        if exc[0] is None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.store[self.key] = (self.start, end)


_NO_SPAN = contextlib.nullcontext()


class Generator:
    """Continuous batching over one engine."""

    def __init__(self, engine: Engine, max_num_seqs: int = 8, max_tokens_per_step: int = 8192,
                 prefill_chunk: int = 0, run_ahead: bool = True, trace: bool = False):
        """``trace``: keep one record per step (what the plan held, host time,
        device time between CUDA events) for ``write_trace``."""
        host = build.host()
        self.engine = engine
        self.host = host
        max_num_seqs = min(max_num_seqs, engine.manager.max_requests())
        self.scheduler = host.Scheduler(
            engine.manager, host.Limits(max_num_seqs, max_tokens_per_step, prefill_chunk))
        self.stats = GenerationStats()
        self._params: Dict[int, SamplingParams] = {}
        self._started: Dict[int, float] = {}
        self._last: Dict[int, float] = {}
        self._limits: Dict[int, int] = {}          # max_new_tokens by request
        self.run_ahead = run_ahead
        self._ahead = None                         # (plan, logits) of a step already launched
        self._planned = None                       # a plan made but not yet run
        self._host_tokens: Optional[torch.Tensor] = None
        self._tokens_copied: Optional[torch.cuda.Event] = None
        self._timing: Dict[int, GenerationResult] = {}
        self._trace: Optional[List[dict]] = [] if trace else None
        self._trace_origin = time.perf_counter()
        self._launch_events: Dict[int, tuple] = {}   # id(plan) -> CUDA events around its launch

    def add(self, prompt: Sequence[int], max_new_tokens: int, params: SamplingParams = SamplingParams(),
            eos_ids: Sequence[int] = (), ignore_eos: bool = False, deadline_s: Optional[float] = None) -> int:
        """Queues a request. ``deadline_s``: seconds from now after which the
        request leaves with finish_reason "deadline", wherever it then is
        (waiting, in its prompt, decoding), keeping what it has generated."""
        params.validate()
        if deadline_s is not None and not deadline_s > 0:
            raise ValueError("deadline_s must be positive")
        prompt = [int(t) for t in prompt]
        vocab = self.engine.spec.vocab_size
        if not prompt:
            raise ValueError("a prompt needs at least one token")
        if min(prompt) < 0 or max(prompt) >= vocab:
            raise ValueError(f"prompt token ids must lie in 0..{vocab - 1}")
        if len(prompt) + max_new_tokens > self.engine.max_context:
            raise ValueError(f"prompt ({len(prompt)}) plus max_new_tokens ({max_new_tokens}) exceeds "
                             f"the context limit of {self.engine.max_context}")
        code = {"icdf": 0, "race": 1}[params.sampler]
        rid = self.scheduler.add(prompt, int(max_new_tokens), [int(e) for e in eos_ids],
                                 bool(ignore_eos),
                                 self.host.SamplingParams(params.temperature, params.seed,
                                                          params.top_p, params.top_k, code),
                                 0.0 if deadline_s is None else self._clock() + float(deadline_s))
        self._params[rid] = params
        self._limits[rid] = int(max_new_tokens)
        self._timing[rid] = GenerationResult(input_ids=prompt, generated_ids=[], finish_reason="")
        self._started[rid] = time.perf_counter()
        return rid

    _clock = staticmethod(time.perf_counter)   # what deadlines are measured on; a test may set another

    def cancel(self, rid: int) -> None:
        self.scheduler.cancel(rid)

    def idle(self) -> bool:
        return self.scheduler.idle()

    def step(self) -> List:
        """One scheduler iteration; returns the events (id, token, finished,
        finish_reason) of this step.

        While every running request is decoding, the next step is launched
        *ahead*: right after this step's tokens have been picked on the device,
        and before they have reached the host, the engine launches the step
        the scheduler will most likely ask for next (the same requests, one
        position further), fed with those tokens on the device. The host then
        reads the tokens, lets the scheduler finish and plan, and keeps the
        step launched ahead if the plan is the one foreseen; otherwise (a
        request stopped at an end-of-sequence token, pages ran out, a request
        arrived) it is dropped and the plan runs as usual. What a request
        generates is the same either way; the device no longer waits for the
        host between two steps."""
        ahead = self._ahead is not None
        if ahead:
            plan, logits, events_key = self._ahead      # launched during the previous call
            self._ahead = None
        else:
            events_key = None
            if self._planned is not None:
                plan, self._planned = self._planned, None
            else:
                plan = self.scheduler.plan(self._clock())
                self.stats.preemptions += len(plan.preempted)
            if not plan.entries:
                return []
            logits = self._launch(plan)
            events_key = id(plan)
        started = time.perf_counter()
        rows = [self._params[e.id] for e in plan.entries if e.wants_token]
        positions = [e.generated_position for e in plan.entries if e.wants_token]
        foreseen = None
        try:
            tokens: List[int] = []
            if logits is not None:
                picked = pick(logits, rows, positions)
                host_tokens = self._token_buffer(len(rows))
                # The tokens and the status word go to the host on a stream of
                # their own, behind the pick: the copy engine's turn does not
                # stand between this step's last kernel and the next step.
                self._picked.record()
                with torch.cuda.stream(self._reader):
                    self._reader.wait_event(self._picked)
                    self.engine.check_later()                   # the status word rides with the tokens
                    host_tokens.copy_(picked, non_blocking=True)
                    self._tokens_copied.record()
                foreseen = self._launch_ahead(plan, picked)     # the device goes on while the host reads
                self._tokens_copied.synchronize()
                tokens = host_tokens.tolist()
                self.engine.check_now()
            else:
                self.engine.check()
            if any(t < 0 for t in tokens):
                raise RuntimeError("non-finite logits")
        except Exception as error:  # the requests of this step leave with the error
            if foreseen is not None:
                self.engine.drop_ahead(foreseen[0])
            self.scheduler.fail_plan(plan, f"step failed: {error}")
            raise
        events = self.scheduler.update(plan, tokens)
        if foreseen is not None:
            requests, ahead_logits = foreseen
            following = self.scheduler.plan(self._clock())
            self.stats.preemptions += len(following.preempted)
            if (not following.preempted and not following.failed
                    and [e.id for e in following.entries] == requests
                    and all(len(e.tokens) == 1 and e.wants_token for e in following.entries)):
                self.engine.commit_ahead(requests)
                self._ahead = (following, ahead_logits, id(requests))
                self.stats.ahead_kept += 1
            else:
                self.engine.drop_ahead(requests)
                self._planned = following                       # runs in the next call, the usual way
                self.stats.ahead_dropped += 1
        now = time.perf_counter()
        self.stats.steps += 1
        self.stats.decode_tokens += plan.decode_tokens
        self.stats.prefill_tokens += plan.prefill_tokens
        self.stats.step_ms.append((now - started) * 1e3)
        if self._trace is not None:
            self._trace.append({
                "step": self.stats.steps - 1, "host_start": started - self._trace_origin, "host_end": now - self._trace_origin,
                "events": self._launch_events.pop(events_key, None), "requests": len(plan.entries),
                "decode_tokens": plan.decode_tokens, "prefill_tokens": plan.prefill_tokens,
                "preempted": len(plan.preempted), "launched_ahead": ahead,
                "waiting": self.scheduler.num_waiting(), "free_pages": self.engine.manager.free_pages(0)})
            if len(self._launch_events) > 8:
                self._launch_events.clear()   # launches of steps that were dropped
        for event in events:
            result = self._timing[event.id]
            if not result.generated_ids and not result.decode_ms and result.prefill_ms == 0.0:
                result.prefill_ms = (now - self._started[event.id]) * 1e3
            else:
                result.decode_ms.append((now - self._last[event.id]) * 1e3)
            self._last[event.id] = now
        return events

    def _launch(self, plan) -> Optional[torch.Tensor]:
        entries = []
        for entry in plan.entries:
            count = len(entry.tokens)
            entries.append(StepEntry(request=entry.id, tokens=entry.tokens,
                                     want=(count - 1,) if entry.wants_token else (), managed=True))
        try:
            with self._device_span(plan):
                return self.engine.step(entries)
        except Exception as error:
            self.scheduler.fail_plan(plan, f"step failed: {error}")
            raise

    def _device_span(self, key):
        """CUDA events around a step's launches, kept under ``key`` for the trace."""
        return _NO_SPAN if self._trace is None else _DeviceSpan(self._launch_events, id(key))

    def _token_buffer(self, count: int) -> torch.Tensor:
        if self._host_tokens is None or self._host_tokens.numel() < count:
            self._host_tokens = torch.empty(max(count, 64), dtype=torch.int32, pin_memory=True)
            self._tokens_copied = torch.cuda.Event()
            self._picked = torch.cuda.Event()
            self._reader = torch.cuda.Stream(device=self.engine.device)
        return self._host_tokens[:count]

    def _launch_ahead(self, plan, picked: torch.Tensor):
        """Launches the step that follows ``plan`` if it can be foreseen: all
        of the plan's requests decode, none of them reaches its token limit
        with the token just picked, and nobody waits to be admitted. Returns
        (requests, logits) or None."""
        if not self.run_ahead or self.scheduler.num_waiting() or not self.engine.ahead_possible():
            return None
        requests = []
        for entry in plan.entries:
            if not entry.wants_token:
                return None
            # generated_position is the index of the token being picked now
            if entry.generated_position + 1 >= self._limits[entry.id]:
                return None
            requests.append(entry.id)
        with self._device_span(requests):
            logits = self.engine.launch_ahead(requests, picked)
        return None if logits is None else (requests, logits)

    def result(self, rid: int) -> GenerationResult:
        info = self.scheduler.request(rid)
        result = self._timing[rid]
        result.generated_ids = list(info.output)
        result.finish_reason = info.finish_reason
        result.failed = info.failed
        result.preemptions = info.preemptions
        result.cached_tokens = len(info.prompt) + max(len(info.output) - 1, 0)
        return result

    def write_trace(self, path: str) -> None:
        """A Chrome / Perfetto JSON timeline: per step one span of the host
        (track "host") and one of the device between the CUDA events around
        its launches (track "device"), with what the plan held as arguments;
        after the reference's ``--trace-out`` timeline of ``engine.step`` and
        ``engine.prefill`` spans (crates/app/cli/src/cli.rs:70-74,
        crates/app/cli/src/engine_loop.rs:619-628)."""
        if self._trace is None:
            raise ValueError("this generator keeps no trace: build it with trace=True")
        torch.cuda.synchronize(self.engine.device)
        events, origin, device_offset = [], None, 0.0
        for record in self._trace:
            arguments = {k: record[k] for k in ("step", "requests", "decode_tokens", "prefill_tokens", "preempted",
                                                 "launched_ahead", "waiting", "free_pages")}
            events.append({"name": "engine.step", "ph": "X", "pid": 1, "tid": 1, "cat": "host",
                           "ts": record["host_start"] * 1e6,
                           "dur": (record["host_end"] - record["host_start"]) * 1e6, "args": arguments})
            pair = record["events"]
            if pair is None:
                continue
            if origin is None:   # device times are relative to the first step's start, laid at its host time
                origin, device_offset = pair[0], record["host_start"] * 1e6
            arguments = dict(arguments, device_ms=pair[0].elapsed_time(pair[1]))
            name = "engine.prefill" if record["prefill_tokens"] else "engine.decode"
            events.append({"name": name, "ph": "X", "pid": 1, "tid": 2, "cat": "device",
                           "ts": device_offset + origin.elapsed_time(pair[0]) * 1e3,
                           "dur": pair[0].elapsed_time(pair[1]) * 1e3, "args": arguments})
        meta = [{"name": "thread_name", "ph": "M", "pid": 1, "tid": 1, "args": {"name": "host"}},
                {"name": "thread_name", "ph": "M", "pid": 1, "tid": 2, "args": {"name": "device"}}]
        with open(path, "w", encoding="utf-8") as handle:
            json.dump({"traceEvents": meta + events, "displayTimeUnit": "ms"}, handle)

    def run(self, on_token: Optional[Callable] = None) -> None:
        """Steps until nothing waits or runs."""
        while not self.scheduler.idle():
            for event in self.step():
                if on_token is not None:
                    on_token(event.id, event.token, event.finished, event.finish_reason)


def generate(engine: Engine, prompts: Sequence[Sequence[int]], max_new_tokens: int = 32,
             temperature: float = 0.0, seed: int = 0, top_p: float = 1.0, top_k: int = 0,
             sampler: str = "icdf", eos_ids: Optional[Sequence[int]] = None,
             ignore_eos: bool = False, max_num_seqs: int = 8, max_tokens_per_step: int = 8192,
             prefill_chunk: int = 0, run_ahead: bool = True, trace_out: Optional[str] = None,
             deadline_s: Optional[float] = None) -> List[GenerationResult]:
    """Generates for every prompt (lists of token ids) and returns the results
    in the prompts' order. ``temperature`` 0 is greedy; otherwise request i
    draws from (seed, stream i). ``eos_ids`` defaults to the configuration's.
    ``trace_out``: a file for the timeline of the steps (``Generator.write_trace``).
    ``deadline_s``: every request leaves with finish_reason "deadline" that long
    after it was queued, as the reference's --generation-timeout-ms."""
    if eos_ids is None:
        eos_ids = tuple(getattr(engine.config, "eos_token_ids", ()) or ())
    generator = Generator(engine, max_num_seqs=max_num_seqs,
                          max_tokens_per_step=max_tokens_per_step, prefill_chunk=prefill_chunk,
                          run_ahead=run_ahead, trace=trace_out is not None)
    ids = [generator.add(prompt, max_new_tokens,
                         SamplingParams(temperature=temperature, seed=seed, stream=index,
                                        top_p=top_p, top_k=top_k, sampler=sampler),
                         eos_ids=eos_ids, ignore_eos=ignore_eos, deadline_s=deadline_s)
           for index, prompt in enumerate(prompts)]
    generator.run()
    if trace_out is not None:
        generator.write_trace(trace_out)
    return [generator.result(rid) for rid in ids]
