"""Continuous-batching scheduler: admission, chunked prefill, decode-first steps, preemption, prefix
cache with GreedyDual-Size eviction, speculative decoding with exact-match acceptance.

Policy follows the reference's ``crates/blaze/src/sched.rs``: one iteration = every decoding request
plus prefill work up to the chunk budget, cut at prefix-cache points (``step`` :2156); FIFO admission that
reserves KV for the prompt and for the active requests' next rows (``admit`` :1211); recompute preemption
of the newest decoding request under KV pressure, resumed before new admissions (``preempt`` :2036,
``resume_preempted`` :2062); prefix-cache entries worth ``inflation + tokens * usefulness(kind)`` evicted
GreedyDual-Size style (``CacheEntry`` :81, ``lookup`` :1131, ``remember`` :1150); speculative rows are sampled
with the request's own parameters and RNG stream and accepted while they equal the draft (:1625-1667);
draft length chosen by an online cost model (``SpecCost`` :262, ``Acceptance`` :235).
"""
from __future__ import annotations

import collections
import os
import enum
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

import torch

from . import log
from .batch import PAGE, SeqChunk
from .tree import DraftTree, merge_chains
from .engine import Engine, OutOfPages, Seq, Snapshot
from .sampler import Rng, SamplingParams, penalty_edits
from .health import StepShape
from .telemetry import Histogram


class Finish(enum.Enum):
    STOP = "stop"          # eos / stop token / stop string
    LENGTH = "length"      # max_tokens or context limit
    ABORT = "abort"
    ERROR = "error"


@dataclass
class GenEvent:
    request_id: str
    tokens: List[int] = field(default_factory=list)
    logprobs: Optional[List[dict]] = None
    finish: Optional[Finish] = None
    error: Optional[str] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0
    hidden: Optional[torch.Tensor] = None     # embeddings requests
    stopped_on: Optional[int] = None          # the last of ``tokens`` is the end-of-sequence / stop token that ended the generation


@dataclass
class ThinkBudget:
    """After ``budget`` tokens inside a thinking block, force ``closing`` token ids (``server.rs:616-634``)."""
    budget: int
    open_id: int
    close_id: int
    closing: List[int]


@dataclass
class GenRequest:
    request_id: str
    prompt: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    cache_point: Optional[int] = None          # explicit prefix-cache boundary (token count)
    constraint: Optional[object] = None        # structured-output constraint (mask / advance)
    think: Optional[ThinkBudget] = None
    embed_only: bool = False                   # return the final-normed hidden state of the last token
    mm: Optional[object] = None                # multimodal inputs
    sink: Optional[Callable[[GenEvent], None]] = None
    t_submit: float = field(default_factory=time.monotonic)


class SnapKind(enum.Enum):
    POINT = 0     # explicit boundary (e.g. the last <|im_start|>)
    PROMPT = 1    # end of a prompt
    FINISH = 2    # end of a generation


@dataclass
class CacheEntry:
    tokens: Tuple[int, ...]
    snap: Snapshot
    kind: SnapKind
    worth: float
    last_used: float = 0.0
    host_run: Optional[Tuple[int, int]] = None      # (start, count) in the host tier while the pages are not on the device


class Usefulness:
    """(used + 1) / (made + 2) per snapshot kind with 0.98 decay (``sched.rs:139-180``)."""

    def __init__(self):
        self.used = {k: 0.0 for k in SnapKind}
        self.made = {k: 0.0 for k in SnapKind}

    def made_one(self, k: SnapKind):
        self.made[k] = self.made[k] * 0.98 + 1.0
        self.used[k] *= 0.98

    def used_one(self, k: SnapKind):
        self.used[k] += 1.0

    def of(self, k: SnapKind) -> float:
        return (self.used[k] + 1.0) / (self.made[k] + 2.0)


class PrefixCache:
    """Snapshots keyed by their token list; longest strict prefix wins; GreedyDual-Size eviction."""

    def __init__(self, engine: Engine, slots: int = 4, enabled: bool = True, host_pages: int = 0):
        self.engine, self.slots, self.enabled = engine, slots, enabled
        self.entries: List[CacheEntry] = []
        # second tier: snapshots evicted from the device wait in pinned host memory (oldest dropped first)
        self.host = None
        self.host_entries: List[CacheEntry] = []
        self.host_hits = 0
        if enabled and host_pages > 0:
            from .kv_host import HostKVTier
            self.host = HostKVTier(engine.kv, host_pages)
        self.inflation = 0.0
        self.use = Usefulness()
        self.hits = self.lookups = self.hit_tokens = 0

    def lookup(self, prompt: Sequence[int]) -> Optional[CacheEntry]:
        if not self.enabled:
            return None
        self.lookups += 1
        best = None
        n = len(prompt)
        for e in self.entries:
            L = len(e.tokens)
            if L < n and (best is None or L > len(best.tokens)) and tuple(prompt[:L]) == e.tokens:
                best = e
        for e in self.host_entries:
            L = len(e.tokens)
            if L < n and (best is None or L > len(best.tokens)) and tuple(prompt[:L]) == e.tokens:
                best = e
        if best is not None and best.host_run is not None and not self._promote(best):
            best = None                # no device pages for it right now: treat as a miss
        if best is not None:
            self.hits += 1
            self.hit_tokens += len(best.tokens)
            best.last_used = time.monotonic()
            self.use.used_one(best.kind)
            best.worth = self.inflation + len(best.tokens) * self.use.of(best.kind)
        return best

    def remember(self, tokens: Sequence[int], seq: Seq, kind: SnapKind) -> bool:
        """Snapshot ``seq`` at ``len(tokens)`` (must be page aligned and equal to its length for recurrent models)."""
        if not self.enabled or self.slots <= 0:
            return False
        n = len(tokens) - len(tokens) % PAGE
        if n < PAGE:
            return False
        key = tuple(tokens[:n])
        for e in self.entries:
            if e.tokens == key:
                e.last_used = time.monotonic()
                return False
        self.use.made_one(kind)
        worth = self.inflation + n * self.use.of(kind)
        while len(self.entries) >= self.slots:
            victim = self._victim(protect=None, incoming=(kind, worth))
            if victim is None:
                return False
            self.evict(victim)
        try:
            snap = self.engine.snapshot(seq, n, with_state=True)
        except (ValueError, OutOfPages):
            return False
        self.entries.append(CacheEntry(key, snap, kind, worth, time.monotonic()))
        return True

    def _victim(self, protect: Optional[CacheEntry], incoming=None) -> Optional[CacheEntry]:
        """Lowest worth; POINT anchors used recently are protected unless the newcomer is a POINT too."""
        now = time.monotonic()
        cands = [e for e in self.entries if e is not protect]
        if not cands:
            return None

        def key(e):
            guard = 1 if (e.kind == SnapKind.POINT and now - e.last_used < 60.0) else 0
            return (guard, e.worth)
        v = min(cands, key=key)
        if incoming is not None and incoming[0] != SnapKind.POINT and v.kind == SnapKind.POINT and v.worth > incoming[1]:
            return None
        return v

    def evict(self, e: CacheEntry) -> None:
        self.inflation = max(self.inflation, e.worth)
        self.entries.remove(e)
        if self.host is not None and e.snap.state_row < 0 and e.snap.pages:
            n = len(e.snap.pages)
            while self.host.free_pages < n and self.host_entries:
                old = self.host_entries.pop(0)
                self.host.drop(old.host_run)
            run = self.host.spill(e.snap.pages)
            if run is not None:
                # the copies are queued on the model's stream, so the pages may go back to the allocator right away
                e.host_run = run
                self.engine.release(e.snap)
                self.host_entries.append(e)
                return
        self.engine.release(e.snap)

    def _promote(self, e: CacheEntry) -> bool:
        """Bring a host-resident entry back: new device pages, one copy per layer, and a device slot for it."""
        n = e.host_run[1]
        try:
            pages = self.engine.pages.alloc(n)
        except OutOfPages:
            return False
        self.host.restore(e.host_run, pages)
        self.host.drop(e.host_run)
        self.host_entries.remove(e)
        e.host_run = None
        e.snap = Snapshot(pages=pages, length=e.snap.length, state_row=-1)
        self.host_hits += 1
        while len(self.entries) >= max(self.slots, 1):
            v = self._victim(protect=e)
            if v is None:
                break
            self.evict(v)
        self.entries.append(e)
        return True

    def evict_for_room(self, protect: Optional[CacheEntry]) -> bool:
        v = self._victim(protect)
        if v is None:
            return False
        self.evict(v)
        return True

    def clear(self) -> None:
        for e in list(self.entries):
            self.engine.release(e.snap)
        self.entries = []
        for e in self.host_entries:
            self.host.drop(e.host_run)
        self.host_entries = []


class Acceptance:
    """Per-depth acceptance ratio, 0.9-decayed, shrunk towards the previous depth (``sched.rs:235-255``)."""

    def __init__(self, depth: int = 16):
        self.hit = [0.0] * depth
        self.tried = [0.0] * depth

    def record(self, drafted: int, accepted: int) -> None:
        for d in range(min(drafted, len(self.hit))):
            self.tried[d] = self.tried[d] * 0.9 + 1.0
            self.hit[d] = self.hit[d] * 0.9 + (1.0 if d < accepted else 0.0)

    def rate(self, d: int) -> float:
        return self.rates(d + 1)[d]

    def rates(self, n: int) -> List[float]:
        """Shrunk acceptance rates of depths 0..n-1 (each shrunk towards the depth before it; 0.7 before depth 0)."""
        out, prev = [], 0.7
        for d in range(n):
            if d < len(self.hit):
                prev = (self.hit[d] + 2.0 * prev) / (self.tried[d] + 2.0)
            out.append(prev)
        return out


class SpecCost:
    """Choose draft lengths: greedy marginal allocation by expected gain, keep the prefix of the allocation
    order that maximises tokens/s under measured verify times by row count (``sched.rs:262-321``)."""

    def __init__(self):
        self.step_ms: Dict[int, float] = {}     # rows (bucketed) → EMA of step time

    @staticmethod
    def _bucket(rows: int) -> int:
        b = 1
        while b < rows:
            b *= 2
        return b

    def observe(self, rows: int, ms: float) -> None:
        b = self._bucket(rows)
        self.step_ms[b] = ms if b not in self.step_ms else 0.8 * self.step_ms[b] + 0.2 * ms

    def time_for(self, rows: int) -> float:
        b = self._bucket(rows)
        if b in self.step_ms:
            return self.step_ms[b]
        known = sorted(self.step_ms)
        if not known:
            return 1.0 + 0.001 * rows
        lo = max([k for k in known if k <= b], default=known[0])
        return self.step_ms[lo] * (1.0 + 0.15 * max(0, (b // max(lo, 1)) - 1))

    def choose(self, acc: Sequence[Acceptance], max_draft: Sequence[int]) -> List[int]:
        import heapq
        n = len(acc)
        rates = [acc[i].rates(max_draft[i]) if max_draft[i] > 0 else [] for i in range(n)]
        # greedy marginal allocation: always extend the sequence whose next draft token is most likely to be accepted
        # (ties go to the lower index); a sequence's gain only shrinks as its draft grows, so a heap gives the arg-max order
        heap = [(-rates[i][0], i) for i in range(n) if rates[i]]
        heapq.heapify(heap)
        k = [0] * n
        order: List[int] = []
        gains: List[float] = []
        while heap:
            g, i = heapq.heappop(heap)
            if -g < 0.05:
                break
            order.append(i)
            gains.append(-g)
            k[i] += 1
            if k[i] < len(rates[i]):
                heapq.heappush(heap, (g * rates[i][k[i]], i))
        # pick the prefix of `order` with the best expected tokens per millisecond
        best_rate, best_len = n / self.time_for(n), 0
        exp_tokens = float(n)
        for j, g in enumerate(gains):
            exp_tokens += g
            r = exp_tokens / self.time_for(n + j + 1)
            if r > best_rate:
                best_rate, best_len = r, j + 1
        out = [0] * n
        for i in order[:best_len]:
            out[i] += 1
        return out


def ngram_propose(history: Sequence[int], k: int, min_n: int = 2, max_n: int = 4, window: int = 65536) -> List[int]:
    """Prompt-lookup drafting: longest suffix n-gram seen earlier (most recent occurrence) → following tokens
    (``sched.rs:2450-2474``)."""
    h = history[-window:]
    L = len(h)
    for n in range(min(max_n, L - 1), min_n - 1, -1):
        suf = h[L - n:]
        for start in range(L - n - 1, -1, -1):
            if h[start:start + n] == suf:
                nxt = h[start + n:start + n + k]
                if nxt:
                    return list(nxt)
    return []


def ngram_propose_many(history: Sequence[int], k: int, width: int, min_n: int = 2, max_n: int = 4,
                       window: int = 65536) -> List[List[int]]:
    """Up to ``width`` different continuations of the suffix n-gram: the most recent occurrence first (the chain
    ``ngram_propose`` gives), then earlier occurrences whose next token differs from the ones already taken."""
    h = history[-window:]
    L = len(h)
    out: List[List[int]] = []
    firsts = set()
    for n in range(min(max_n, L - 1), min_n - 1, -1):
        suf = h[L - n:]
        for start in range(L - n - 1, -1, -1):
            if h[start:start + n] == suf:
                nxt = list(h[start + n:start + n + k])
                if nxt and nxt[0] not in firsts:
                    firsts.add(nxt[0])
                    out.append(nxt)
                    if len(out) >= width:
                        return out
        if out:
            break                      # alternatives come from the same (longest matching) n-gram order
    return out


@dataclass
class SchedConfig:
    chunk: int = 2048                  # prefill tokens per iteration
    max_step_tokens: int = 8192
    max_seqs: int = 256
    prefix_cache: bool = True
    cache_slots: int = 4
    spec_method: str = "none"          # none | ngram | suffix | mtp | eagle
    max_draft: int = 4
    max_verify: int = 8
    spec_fixed: bool = False           # verify every draft at full length instead of asking the cost model
    draft_tree_width: int = 1          # > 1: n-gram drafts branch into up to this many continuations, verified as a tree
    uniform_verify: bool = True        # pad chain drafts to one length when the verify step can then replay a captured graph
    draft_tree_depth: int = 4          # deepest level of a draft tree (n-gram continuations are cut, drafter trees grown, to it)
    eos_ids: Tuple[int, ...] = ()
    max_model_len: int = 4096
    # "interleave": every step takes all decoding requests plus at most one prefill chunk (steady token flow for running
    # requests); "prefill_first": while prompts are waiting to be read, steps carry prefill chunks only and decoding
    # requests join at most every `max_decode_stall` seconds (higher throughput and earlier first tokens under bursts)
    schedule: str = "interleave"
    max_decode_stall: float = 0.25
    kv_host_pages: int = 0             # pinned host pages behind the prefix cache (0 = no host tier)
    run_ahead: bool = True             # launch greedy decode step k+1 before reading step k (tokens fed back on the device)


@dataclass
class SchedStats:
    steps: int = 0
    prompt_tokens: int = 0
    cached_tokens: int = 0
    output_tokens: int = 0
    preemptions: int = 0
    draft_tokens: int = 0
    accepted_tokens: int = 0
    finished: int = 0
    failed: int = 0


class Active:
    def __init__(self, req: GenRequest, seq: Seq, cached: int):
        self.req, self.seq = req, seq
        self.tokens: List[int] = list(req.prompt)     # prompt + generated
        self.n_prompt = len(req.prompt)
        self.computed = cached                         # tokens whose KV is in the cache
        self.cached = cached
        self.rng = Rng(req.params.seed if req.params.seed is not None else (hash(req.request_id) & 0xFFFFFFFF))
        self.acc = Acceptance()
        self.t_first = 0.0
        self.t_last = 0.0
        self.think_used = -1
        self.forced: Deque[int] = collections.deque()
        self.admitted_at = time.monotonic()
        self.snap_points: List[int] = []
        # multimodal requests: rotary positions of the prompt rows (3 x prompt) and what text rows after it add to their index
        self.mm_pos = None
        self.rope_delta = 0
        self.cache_key_tokens: Optional[List[int]] = None     # prompt with image pads replaced by content keys
        if req.mm is not None:
            self.mm_pos = req.mm.positions3(self.tokens[:self.n_prompt])
            self.rope_delta = int(self.mm_pos.max().item()) + 1 - self.n_prompt if self.n_prompt else 0
            self.cache_key_tokens = req.mm.cache_tokens(self.tokens[:self.n_prompt])

    @property
    def generated(self) -> List[int]:
        return self.tokens[self.n_prompt:]

    @property
    def decoding(self) -> bool:
        return self.computed >= len(self.tokens) - 1 and len(self.tokens) > self.n_prompt - 1 and self.computed >= self.n_prompt - 1 and self._started

    _started = False


class _Ahead:
    """A greedy decode step that was launched but whose tokens the host has not read yet."""
    __slots__ = ("actives", "tokens", "event", "t0")

    def __init__(self, actives, tokens, event, t0):
        self.actives, self.tokens, self.event, self.t0 = actives, tokens, event, t0


class _Pending:
    """A launched step whose results the host has not consumed yet."""
    __slots__ = ("plan", "mode", "out", "t0", "seen", "host", "event", "real_k")

    def __init__(self, plan, mode, out, t0):
        self.plan, self.mode, self.out, self.t0 = plan, mode, out, t0
        self.real_k: Dict[int, int] = {}  # request -> length of its own draft when the drafts were padded to one length
        self.seen: List[tuple] = []      # (request, first row, first position, rows)
        self.host = None                 # pinned copy of the greedy tokens when the step is left in flight
        self.event = None


class Scheduler:
    def __init__(self, engine: Engine, cfg: SchedConfig, drafter=None, sample_fn=None):
        self.engine, self.cfg, self.drafter = engine, cfg, drafter
        self.waiting: Deque[GenRequest] = collections.deque()
        self.preempted: Deque[Active] = collections.deque()
        self.active: List[Active] = []
        self.cache = PrefixCache(engine, cfg.cache_slots, cfg.prefix_cache, cfg.kv_host_pages)
        self.stats = SchedStats()
        self.cost = SpecCost()
        self.inbox: "queue.Queue[GenRequest]" = queue.Queue()
        self.aborts: "queue.Queue[str]" = queue.Queue()
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.ttft = Histogram.latency()
        self.tpot = Histogram.latency()
        self.step_ms = Histogram.latency()
        self.sample_fn = sample_fn
        self.on_step: Optional[Callable[[float, int], None]] = None
        self._ahead: Optional[_Ahead] = None
        self._pending: Optional[_Pending] = None
        self._last_decode = 0.0
        self._cuda_sampler = None
        ops = getattr(getattr(engine, "model", None), "ops", None)
        if ops is not None and getattr(ops, "is_cuda", False) and sample_fn is None and os.environ.get("BLAZE_CUDA_SAMPLER", "1") != "0":
            from .sampler_cuda import CudaSampler
            self._cuda_sampler = CudaSampler(ops)
        from .suffix import SuffixIndex
        self.suffix = SuffixIndex() if cfg.spec_method == "suffix" else None
        from .health import Health
        self.health = Health()
        self.raise_step_errors = False     # debugging aid: let a failing step raise instead of failing its requests

    # ================================================================== public
    def submit(self, req: GenRequest) -> None:
        self.inbox.put(req)

    def abort(self, request_id: str) -> None:
        self.aborts.put(request_id)

    #: (every n steps, callable) pairs run on the scheduler thread between steps (statistics that must not race the GPU work)
    housekeeping: tuple = ()

    def start(self) -> None:
        self._thread = threading.Thread(target=self._loop, name="blaze-sched", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=10)

    @property
    def idle(self) -> bool:
        return not (self.active or self.waiting or self.preempted or self._ahead or self._pending) and self.inbox.empty()

    def run_until_idle(self, max_steps: int = 1 << 30) -> None:
        n = 0
        while not self.idle and n < max_steps:
            self.safe_step()
            n += 1

    def safe_step(self) -> None:
        """One step; a step that fails (a kernel reported an error through the device status word, a sampler error, an
        exception in the model) fails the requests that were running and leaves the scheduler ready for the next ones
        (``crates/blaze/src/sched.rs:1067-1075``)."""
        try:
            self.step()
            for every, fn in self.housekeeping:
                if self.stats.steps % every == 0:
                    fn()
        except Exception as e:
            if self.raise_step_errors:
                raise
            log.error("sched.step_failed", error=repr(e))
            self._ahead = self._pending = None
            blamed = list(self.active)
            for a in blamed:
                self._retire(a, Finish.ERROR, error=repr(e))
            if not blamed:
                # the failure came before any request ran (admission): fail the request at the head of the queue, so that a
                # failure that repeats cannot keep the loop spinning on the same request
                if self.preempted:
                    a = self.preempted.popleft()
                    self._emit(a, GenEvent(a.req.request_id, finish=Finish.ERROR, error=repr(e), prompt_tokens=a.n_prompt))
                elif self.waiting:
                    req = self.waiting.popleft()
                    self._emit(req, GenEvent(req.request_id, finish=Finish.ERROR, error=repr(e), prompt_tokens=len(req.prompt)))
            self.stats.failed += 1
            self.health.errors += 1

    def _loop(self) -> None:
        while not self._stop.is_set():
            if self.idle:
                try:
                    self.waiting.append(self.inbox.get(timeout=0.05))
                except queue.Empty:
                    continue
            self.safe_step()
            self.health.tick(active=len(self.active), waiting=len(self.waiting), kv_pages_free=self.engine.pages.free_count)

    # ================================================================== admission
    def _reserved(self) -> int:
        r = 0
        for a in self.active:
            r += max(self.cfg.max_verify if self.cfg.spec_method != "none" else 1, len(a.tokens) - a.computed) + PAGE
        return r

    def _emit(self, a_or_req, ev: GenEvent) -> None:
        req = a_or_req.req if isinstance(a_or_req, Active) else a_or_req
        if req.sink:
            try:
                req.sink(ev)
            except Exception as e:   # a consumer that went away must not take the step down with it
                log.debug("sched.sink_failed", request_id=req.request_id, error=repr(e))

    def _admit(self) -> None:
        while True:
            try:
                self.waiting.append(self.inbox.get_nowait())
            except queue.Empty:
                break
        while True:
            try:
                rid = self.aborts.get_nowait()
            except queue.Empty:
                break
            for a in list(self.active):
                if a.req.request_id == rid:
                    self._retire(a, Finish.ABORT)
            self.waiting = collections.deque(r for r in self.waiting if r.request_id != rid)
        # preempted requests come back before new admissions
        while self.preempted and self._try_admit(self.preempted[0].req, resume=self.preempted[0]):
            self.preempted.popleft()
        while self.waiting and not self.preempted:
            req = self.waiting[0]
            ok = self._try_admit(req)
            if ok is None:
                self.waiting.popleft()     # rejected with an error event
                continue
            if not ok:
                break
            self.waiting.popleft()

    def _try_admit(self, req: GenRequest, resume: Optional[Active] = None):
        eng = self.engine
        if req.mm is not None and not resume and not getattr(req, "_mm_expanded", False):
            # one placeholder per image in the rendered prompt becomes as many pad tokens as the image has embedding rows
            if sum(1 for t in req.prompt if t == req.mm.image_pad_id) == len(req.mm.images):
                req.prompt = req.mm.expand(req.prompt)
            req._mm_expanded = True
        tokens = resume.tokens if resume else req.prompt
        if len(self.active) >= self.cfg.max_seqs or not eng.free_rows:
            return False
        if not tokens:
            self._emit(req, GenEvent(req.request_id, finish=Finish.ERROR, error="empty prompt"))
            return None
        limit = min(self.cfg.max_model_len, eng.max_pages_per_seq * PAGE)
        if len(tokens) + 1 > limit:
            self._emit(req, GenEvent(req.request_id, finish=Finish.ERROR,
                                     error=f"prompt of {len(tokens)} tokens exceeds the context limit {limit}"))
            self.stats.failed += 1
            return None
        # images take part in prefix matching through their content keys, not through the (identical) pad tokens
        key_tokens = req.mm.cache_tokens(tokens) if req.mm is not None else tokens
        entry = self.cache.lookup(key_tokens)
        cached = len(entry.tokens) if entry else 0
        need = len(tokens) - cached + 16 + self._reserved()
        while eng.free_tokens < need:
            if not self.cache.evict_for_room(protect=entry):
                break
        if eng.free_tokens < need:
            if not self.active and not self.cache.entries:
                self._emit(req, GenEvent(req.request_id, finish=Finish.ERROR, error="prompt can never fit the KV pool"))
                self.stats.failed += 1
                return None
            return False
        seq = eng.open_from(entry.snap if entry else None)
        if resume:
            a = resume
            a.seq, a.computed, a.cached = seq, cached, cached
        else:
            a = Active(req, seq, cached)
            self.stats.prompt_tokens += len(tokens)
        self.stats.cached_tokens += cached
        # prefill cut points: explicit cache point and the page-aligned end of the prompt
        pts = []
        if req.cache_point and cached < req.cache_point < len(tokens):
            pts.append(req.cache_point - req.cache_point % PAGE)
        end = (a.n_prompt - 1) - (a.n_prompt - 1) % PAGE
        if end > cached:
            pts.append(end)
        a.snap_points = sorted(set(p for p in pts if p > cached))
        self.active.append(a)
        if self.drafter is not None and hasattr(self.drafter, "open"):
            self.drafter.close(req.request_id)
            self.drafter.open(req.request_id)
            if cached:
                # the drafter has no state for a cached prefix: it starts drafting from what it sees from here on
                self.drafter.states[req.request_id].fed = cached
                try:
                    self.drafter.engine.reserve(self.drafter.states[req.request_id].seq, cached)
                    self.drafter.states[req.request_id].seq.length = cached
                except Exception:
                    pass
        return True

    # ================================================================== preemption
    def _preempt_newest(self, keep: Optional[Active] = None) -> bool:
        cands = [a for a in self.active if a is not keep]
        if not cands:
            return False
        a = max(cands, key=lambda x: x.admitted_at)
        self.engine.close(a.seq)
        self.active.remove(a)
        a.seq = None
        a.computed = 0
        a._started = False
        self.preempted.append(a)
        if self.drafter is not None and hasattr(self.drafter, "close"):
            self.drafter.close(a.req.request_id)
        self.stats.preemptions += 1
        log.debug("sched.preempt", request_id=a.req.request_id, tokens=len(a.tokens))
        return True

    # ================================================================== one iteration
    # ================================================================== run-ahead decode
    # While every active request is a plain greedy decoder, the next step's input tokens are this step's output, and they
    # are already on the device.  So step k+1 is launched (tokens fed back on the device) before the host reads step k:
    # the host's bookkeeping for step k then overlaps the GPU's work on step k+1.  A request that stops on a token the
    # host had not seen yet (EOS) has taken part in one step too many; its row is ignored and its pages are released
    # — later owners of those pages write them after that step in stream order.
    def _plain_greedy(self, a: Active) -> bool:
        p, r = a.req.params, a.req
        return not (p.needs_candidates() or r.constraint is not None or r.embed_only or r.think is not None or a.forced
                    or p.logprobs is not None or r.mm is not None)

    def _continues(self, a: Active, in_flight: int) -> bool:
        """True when ``a`` certainly wants another token after the ``in_flight`` tokens that are not appended yet."""
        n = len(a.tokens) + in_flight
        limit = min(self.cfg.max_model_len, self.engine.max_pages_per_seq * PAGE)
        return n - a.n_prompt < a.req.params.max_tokens and n + 1 < limit

    def _hand_off(self, actives: List[Active], out: torch.Tensor, t0: float) -> _Ahead:
        if out.device.type == "cuda":
            host = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
            host.copy_(out, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        else:
            host, ev = out.clone(), None
        self.engine.d2h_bytes += out.numel() * out.element_size()
        return _Ahead(actives, host, ev, t0)

    def _launch_ahead(self, actives: List[Active]) -> Optional[_Ahead]:
        eng = self.engine
        t0 = time.monotonic()
        try:
            for a in actives:
                eng.reserve(a.seq, a.computed + 2)
        except OutOfPages:
            return None
        chunks = []
        for a in actives:
            chunks.append(SeqChunk(slot=a.seq.row, tokens=[0], start_pos=a.computed + 1, want_logits=1))
            a.seq.length = a.computed + 2
        out = eng.forward(chunks, "greedy", feedback=True)
        return self._hand_off(actives, out, t0)

    def _consume_ahead(self, ah: _Ahead) -> None:
        if ah.event is not None:
            ah.event.synchronize()
        self.engine.check_status()
        toks = ah.tokens.tolist()
        n = 0
        for a, tok in zip(ah.actives, toks):
            if a.seq is None:           # stopped, aborted or preempted while the step was in flight
                continue
            a.computed += 1
            a._started = True
            n += 1
            self._append(a, [tok], [])
        dt = (time.monotonic() - ah.t0) * 1e3
        self.step_ms.observe(dt / 1e3)
        self.stats.steps += 1
        self.health.step(dt / 1e3, StepShape(rows=n, seqs=n))
        if self.on_step:
            self.on_step(dt, n)

    def _step_ahead(self) -> None:
        ah = self._ahead
        self._admit()
        nxt = None
        same = len(self.active) == len(ah.actives) and all(x is y for x, y in zip(self.active, ah.actives))
        if same and all(self._continues(a, 1) for a in ah.actives):
            nxt = self._launch_ahead(ah.actives)
        self._ahead = None
        self._consume_ahead(ah)
        self._ahead = nxt

    def step(self) -> None:
        if self._ahead is not None:
            return self._step_ahead()
        self._admit()
        if not self.active:
            return
        eng, cfg = self.engine, self.cfg
        t0 = time.monotonic()
        # ---- plan rows: decoding requests first, then prefill work within the chunk budget
        plan: List[Tuple[Active, List[int], int, List[int]]] = []   # (active, tokens, want_logits, draft)
        budget = cfg.max_step_tokens
        decoders = [a for a in self.active if a.computed == len(a.tokens) - 1 and a.computed >= a.n_prompt - 1]
        if cfg.schedule == "prefill_first" and decoders and len(decoders) < len(self.active):
            if t0 - self._last_decode < cfg.max_decode_stall:
                decoders = []            # prompts first; the running requests wait a bounded time
        if decoders:
            self._last_decode = t0
        spec = cfg.spec_method != "none" and decoders
        drafts: Dict[int, List[int]] = {}
        real_k: Dict[int, int] = {}
        if spec:
            drafts = self._draft(decoders)
            real_k = self._pad_drafts(decoders, drafts)
        for a in decoders:
            d = drafts.get(id(a), [])
            drafted = d.token[1:] if isinstance(d, DraftTree) else d
            plan.append((a, [a.tokens[-1]] + list(drafted), 1 + len(drafted), d))
            budget -= 1 + len(drafted)
        chunk_left = min(cfg.chunk, max(budget, 0))
        dec_ids = {id(a) for a in decoders}
        for a in self.active:
            if id(a) in dec_ids or chunk_left <= 0:
                continue
            remaining = len(a.tokens) - a.computed
            if remaining <= 0 or (remaining <= 1 and a.computed >= a.n_prompt - 1):
                continue                 # its last step is still in flight, or a decoding request that sits this step out
            n = min(remaining, chunk_left)
            for pt in a.snap_points:
                if a.computed < pt < a.computed + n:
                    n = pt - a.computed
                    break
            last = a.computed + n == len(a.tokens)
            plan.append((a, a.tokens[a.computed:a.computed + n], 1 if last else 0, []))
            chunk_left -= n
        if not plan:
            if self._pending is not None:
                prev, self._pending = self._pending, None
                self._consume(prev)
            return
        # ---- KV room (recompute-preempt the newest request when pages run out)
        while True:
            try:
                items = []
                for a, toks, want, _ in plan:
                    eng.reserve(a.seq, a.computed + len(toks))
                    items.append((a.seq, toks, want))
                break
            except OutOfPages:
                if self.cache.evict_for_room(None):
                    continue
                victim_ok = self._preempt_newest(keep=plan[0][0] if len(plan) == 1 else None)
                if not victim_ok:
                    a = plan[0][0]
                    self._retire(a, Finish.LENGTH)
                    return
                plan = [p for p in plan if p[0] in self.active]
                if not plan:
                    return
        for a, toks, _, _ in plan:
            a.seq.length = a.computed            # plan() advances from here
        chunks = []
        for (a, toks, want, d) in plan:
            if isinstance(d, DraftTree):
                chunks += eng.plan_tree([(a.seq, toks, d.parent)])
            else:
                chunks += eng.plan([(a.seq, toks, want)], defer_state=bool(d))
            self._mm_fill(a, chunks[-1])
        want_any = any(w for _, _, w, _ in plan)
        need_logits = any(w and (a.req.params.needs_candidates() or a.req.constraint is not None or a.req.embed_only)
                          for a, _, w, _ in plan)
        mode = "none" if not want_any else ("both" if any(a.req.embed_only for a, _, w, _ in plan if w) else
                                            ("logits" if need_logits else "greedy"))
        if self.drafter is not None and mode in ("greedy", "logits"):
            mode = "greedy_hidden" if mode == "greedy" else "both"      # the drafter reads the target's hidden rows
        out = eng.forward(chunks, mode)
        if (mode == "greedy" and cfg.run_ahead and len(plan) == len(self.active) and all(len(t) == 1 for _, t, _, _ in plan)
                and eng.can_feed_back(len(plan)) and all(self._plain_greedy(a) and self._continues(a, 1) for a, _, _, _ in plan)):
            self._ahead = self._hand_off([a for a, _, _, _ in plan], out, t0)
            return
        pend = _Pending(plan, mode, out, t0)
        pend.real_k = real_k
        self._advance(pend)
        # The step before this one may still be unread: its results are taken now, while the GPU works on the new step.
        prev, self._pending = self._pending, None
        if prev is not None:
            self._consume(prev)
        if self._may_stay_in_flight(pend):
            if mode == "greedy":
                if out.device.type == "cuda":
                    pend.host = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
                    pend.host.copy_(out, non_blocking=True)
                    pend.event = torch.cuda.Event()
                    pend.event.record()
                else:
                    pend.host = out.clone()
            self._pending = pend
        else:
            self._consume(pend)

    def _key_tokens(self, a: Active, n: int) -> List[int]:
        """The first ``n`` tokens of ``a`` as the prefix cache sees them (image pads replaced by image content keys)."""
        if a.cache_key_tokens is None:
            return a.tokens[:n]
        k = a.cache_key_tokens
        return k[:n] if n <= len(k) else k + a.tokens[len(k):n]

    def _mm_fill(self, a: Active, ch: SeqChunk) -> None:
        """Rotary positions and image-embedding rows of a chunk of a multimodal request."""
        if a.req.mm is None:
            return
        n, p0 = len(ch.tokens), ch.start_pos
        ch.rope_delta = a.rope_delta
        if p0 < a.n_prompt:
            m = min(n, a.n_prompt - p0)
            pos = torch.empty(3, n, dtype=torch.int32)
            pos[:, :m] = a.mm_pos[:, p0:p0 + m]
            if n > m:
                pos[:, m:] = torch.arange(p0 + m, p0 + n, dtype=torch.int32) + a.rope_delta
            ch.pos3 = pos.tolist()
            blocks = []
            for s0, e0, k in a.req.mm.segments(a.tokens[:a.n_prompt]):
                lo, hi = max(s0, p0), min(e0, p0 + n)
                if lo < hi and k < len(a.req.mm.images):
                    blocks.append((lo - p0, a.req.mm.images[k].embeds[lo - s0:hi - s0]))
            ch.embeds = blocks or None

    def _may_stay_in_flight(self, pend: "_Pending") -> bool:
        """Plain greedy / headless steps without drafts: nothing the host decides next depends on their tokens, except
        for the requests in the step themselves, and those sit out until the tokens are read."""
        if not self.cfg.run_ahead or self.drafter is not None or pend.mode not in ("greedy", "none"):
            return False
        if pend.out is not None and pend.out.device.type != "cuda":
            return self.engine.ecfg.feedback_eager          # CPU tests of the overlap logic
        if pend.out is None and self.engine.device.type != "cuda":
            return self.engine.ecfg.feedback_eager
        # decode rows would have to sit out the next step (their token is not read yet): only prompt chunks stay in flight
        if any(p0 >= a.n_prompt - 1 for a, _, p0, _ in pend.seen):
            return False
        return all(not d and (w == 0 or self._plain_greedy(a)) for a, _, w, d in pend.plan)

    def _advance(self, pend: "_Pending") -> None:
        """Book the step's rows as computed (and take the prefix-cache snapshots that fall on its end) at launch time."""
        row0 = 0
        for a, toks, want, draft in pend.plan:
            pend.seen.append((a, row0, a.computed, len(toks)))
            row0 += len(toks)
            a.computed += len(toks)
            a._started = True
            if a.computed in a.snap_points and a.computed <= a.n_prompt:
                kind = SnapKind.POINT if a.req.cache_point and a.computed <= a.req.cache_point else SnapKind.PROMPT
                self.cache.remember(self._key_tokens(a, a.computed), a.seq, kind)

    def _consume(self, pend: "_Pending") -> None:
        eng = self.engine
        plan, mode, out, t0 = pend.plan, pend.mode, pend.out, pend.t0
        # ---- consume results
        row = 0
        rows_total = sum(len(t) for _, t, _, _ in plan)
        host_tokens = None
        logits = hidden = None
        if mode == "greedy_hidden":
            out, hidden = out
            mode = "greedy"
        if mode == "greedy":
            if pend.host is not None:
                if pend.event is not None:
                    pend.event.synchronize()
                host_tokens = pend.host.tolist()
            else:
                host_tokens = out.tolist()
            eng.d2h_bytes += out.numel() * out.element_size()
        elif mode == "logits":
            logits = out
        elif mode == "both":
            logits, hidden = out
        if mode != "greedy" and out is not None and eng.device.type == "cuda":
            torch.cuda.current_stream(eng.device).synchronize()     # logits / hidden rows are read on the host next
        if mode != "none":
            eng.check_status()       # the step's results are on their way to the host: was any of its kernels in trouble?
        # rows whose chain the batched CUDA sampler covers are drawn with one launch and one copy for the whole step
        pre: Dict[int, object] = {}
        if logits is not None and self._cuda_sampler is not None:
            from .sampler_cuda import eligible
            picks, rows_in, r = [], [], 0
            for a, toks, want, draft in plan:
                if want == 1 and not a.req.embed_only and not a.forced and eligible(a.req.params):
                    p = a.req.params
                    edits = penalty_edits(p, a.tokens[:a.n_prompt], a.generated, self.cfg.eos_ids) \
                        if (p.has_penalties() or p.logit_bias) else {}
                    allowed = a.req.constraint.mask([]) if a.req.constraint is not None else None
                    picks.append(a)
                    rows_in.append((p, a.rng.uniform(), edits, allowed))
                    r_idx = r
                    rows_in[-1] = rows_in[-1] + (r_idx,)
                r += want
            if picks:
                idx = torch.tensor([x[4] for x in rows_in], device=logits.device)
                res = self._cuda_sampler.sample(logits.index_select(0, idx).contiguous(), [x[:4] for x in rows_in],
                                                self.engine.model.cfg.vocab_size)
                eng.d2h_bytes += len(picks) * (8 + 4 * 130)
                for a, rr in zip(picks, res):
                    pre[id(a)] = rr
        seen = pend.seen
        for a, toks, want, draft in plan:
            if not want:
                continue
            if a.seq is None:            # aborted or preempted while the step was in flight
                row += want
                continue
            if a.req.embed_only:
                from .batch import StepBatch  # noqa: F401
                h = eng.model.final_hidden(hidden, torch.tensor([eng_row_index(plan, a)], device=hidden.device))
                self._emit(a, GenEvent(a.req.request_id, hidden=h[0].float().cpu(), prompt_tokens=a.n_prompt,
                                       cached_tokens=a.cached))
                self._retire(a, Finish.STOP, silent=True)
                row += want
                continue
            new: List[int] = []
            lps: List[dict] = []
            accepted = 0
            if isinstance(draft, DraftTree):
                # walk from the root: sample the row of the current node, follow the child that drafted that token
                node, path = 0, []
                while True:
                    if host_tokens is not None:
                        tok, lp = host_tokens[row + node], None
                    else:
                        tok, lp = self._sample(a, logits[row + node], new)
                    new.append(tok)
                    if lp is not None:
                        lps.append(lp)
                    node = next((c for c in draft.children(node) if draft.token[c] == tok), None)
                    if node is None:
                        break
                    path.append(node)
                row += want
                depth = max((draft.depth(i) for i in range(len(draft.token))), default=0)
                a.acc.record(depth, len(path))
                self.stats.draft_tokens += len(draft.token) - 1
                self.stats.accepted_tokens += len(path)
                base = a.computed - len(toks)
                eng.commit_tree([(a.seq, base, path)])       # accepted rows move into place, the other branches go
                a.computed = base + 1 + len(path)
                self._append(a, new, lps)
                continue
            for j in range(want):
                if a.forced:
                    tok, lp = a.forced.popleft(), None
                elif host_tokens is not None:
                    tok, lp = host_tokens[row + j], None
                elif id(a) in pre:
                    tok, lp = self._take_presampled(a, pre.pop(id(a)))
                else:
                    tok, lp = self._sample(a, logits[row + j], new)
                new.append(tok)
                if lp is not None:
                    lps.append(lp)
                if j < len(draft) and tok == draft[j]:
                    accepted += 1
                    continue
                break
            row += want
            if draft:
                # chains padded to one length for a captured verify step: only the drafter's own tokens count as drafted
                real = pend.real_k.get(id(a), len(draft)) if pend.real_k else len(draft)
                if real:
                    a.acc.record(real, min(accepted, real))
                self.stats.draft_tokens += real
                self.stats.accepted_tokens += min(accepted, real)
                # KV of rejected draft rows is dropped; the last emitted token's KV is computed next step
                a.computed = a.computed - len(toks) + 1 + accepted
                if eng.kv.gdn_layers:
                    eng.commit_state([(a.seq, 1 + accepted)])     # recurrent layers advance over the accepted rows only
                eng.truncate(a.seq, a.computed)
            self._append(a, new, lps)
        if self.drafter is not None and hidden is not None:
            if hasattr(self.drafter, "hidden_source"):
                hidden = self.drafter.hidden_source(eng.model, hidden)
            for a, r0, p0, n in seen:
                if a.seq is None or a.req.embed_only:
                    continue
                keep = min(n, a.computed - p0, len(a.tokens) - 1 - p0)     # rows whose KV survived and whose next token is known
                if keep > 0:
                    self.drafter.observe(a.req.request_id, hidden[r0:r0 + keep], a.tokens[p0 + 1:p0 + 1 + keep], p0)
        dt = (time.monotonic() - t0) * 1e3
        self.cost.observe(rows_total, dt)
        self.step_ms.observe(dt / 1e3)
        self.stats.steps += 1
        self.health.step(dt / 1e3, StepShape(rows=rows_total, seqs=len(plan)))
        if self.on_step:
            self.on_step(dt, rows_total)

    # ------------------------------------------------------------------ helpers
    def _pad_drafts(self, decoders: List[Active], drafts: Dict[int, List[int]]) -> Dict[int, int]:
        """Make a chain-verify step uniform so that it can replay a captured graph: when every running request decodes, all
        sample greedily and the engine can capture ``len(decoders) x (k + 1)`` rows, every draft is padded to the longest
        one with filler tokens (verification rejects them like any wrong draft; the rare filler that happens to be right is
        simply accepted).  Returns the drafts' own lengths by request (empty when nothing was padded)."""
        eng, cfg = self.engine, self.cfg
        if not cfg.uniform_verify or not drafts or len(decoders) != len(self.active) or not hasattr(eng, "verify_graphable"):
            return {}
        if any(isinstance(d, DraftTree) for d in drafts.values()):
            return {}
        k = max(len(d) for d in drafts.values())
        if k <= 0 or not eng.verify_graphable(len(decoders), k + 1):
            return {}
        limit = min(cfg.max_model_len, eng.max_pages_per_seq * PAGE)
        for a in decoders:
            room = a.req.params.max_tokens - len(a.generated) - 1
            if (room < k or len(a.tokens) + k + 1 > limit or not self._plain_greedy(a) or a.req.constraint is not None or a.forced
                    or a.req.embed_only or a.req.mm is not None):
                return {}
        real = {}
        for a in decoders:
            d = list(drafts.get(id(a), []))
            real[id(a)] = len(d)
            if len(d) < k:
                d += [d[-1] if d else a.tokens[-1]] * (k - len(d))
            drafts[id(a)] = d
        return real

    def _draft(self, decoders: List[Active]) -> Dict[int, List[int]]:
        cfg = self.cfg
        maxd = []
        for a in decoders:
            room = a.req.params.max_tokens - len(a.generated) - 1
            ok = a.req.constraint is None and not a.forced
            maxd.append(max(0, min(cfg.max_draft, room)) if ok else 0)
        # spec_fixed: always verify the whole draft; else drafts are cut or skipped by the measured verify cost
        want = list(maxd) if cfg.spec_fixed else self.cost.choose([a.acc for a in decoders], maxd)
        out: Dict[int, List[int]] = {}
        if cfg.spec_method == "ngram":
            eng = self.engine
            group = max(eng.model.cfg.num_heads // max(eng.model.cfg.num_kv_heads, 1), 1)
            tree_rows = min(32, max(64 // group, 1)) if (cfg.draft_tree_width > 1 and not eng.kv.gdn_layers) else 0
            for a, k in zip(decoders, want):
                if k <= 0:
                    continue
                if tree_rows > 2:
                    chains = ngram_propose_many(a.tokens, k, cfg.draft_tree_width)
                    if len(chains) > 1:
                        out[id(a)] = merge_chains(chains, tree_rows)
                        continue
                    d = chains[0] if chains else []
                else:
                    d = ngram_propose(a.tokens, k)
                if d:
                    out[id(a)] = d
        elif cfg.spec_method == "suffix" and self.suffix is not None:
            for a, k in zip(decoders, want):
                if k > 0:
                    d = self.suffix.draft(a.tokens, k)
                    if d:
                        out[id(a)] = d
        elif self.drafter is not None:
            reqs = [(a, k) for a, k in zip(decoders, want) if k > 0]
            if reqs and cfg.draft_tree_width > 1 and hasattr(self.drafter, "propose_tree") and not self.engine.kv.gdn_layers:
                # trees grown by the drafter itself (EAGLE): verified with the tree rows of the target's attention
                eng = self.engine
                group = max(eng.model.cfg.num_heads // max(eng.model.cfg.num_kv_heads, 1), 1)
                cap = min(32, max(64 // group, 1), cfg.max_verify)
                ts = self.drafter.propose_tree([a for a, _ in reqs], cfg.draft_tree_width, min(cfg.draft_tree_depth, cfg.max_draft), cap)
                for (a, _), t in zip(reqs, ts):
                    if t is not None:
                        out[id(a)] = t
            elif reqs:
                ds = self.drafter.propose([a for a, _ in reqs], [k for _, k in reqs])
                for (a, _), d in zip(reqs, ds):
                    if d:
                        out[id(a)] = list(d)
        return out

    def _sample(self, a: Active, logits_row: torch.Tensor, pending: List[int]):
        p = a.req.params
        edits = penalty_edits(p, a.tokens[:a.n_prompt], a.generated, self.cfg.eos_ids, draft_prefix=pending) \
            if (p.has_penalties() or p.logit_bias) else {}
        allowed = a.req.constraint.mask(pending) if a.req.constraint is not None else None
        draw = a.rng.uniform()
        fn = self.sample_fn
        if fn is None:
            from .sampler_torch import sample_row
            fn = sample_row
        res = fn(logits_row, p, draw, edits, allowed, self.engine.model.cfg.vocab_size)
        if res.status != 0:
            raise RuntimeError(f"sampler status {res.status} for request {a.req.request_id}")
        lp = None
        if p.logprobs is not None:
            lp = {"token": res.token, "logprob": res.logprob, "top": res.top[:p.logprobs]}
        if a.req.constraint is not None:
            a.req.constraint.advance(res.token)
        return res.token, lp

    def _take_presampled(self, a: Active, res):
        if res.status != 0:
            raise RuntimeError(f"sampler status {res.status} for request {a.req.request_id}")
        p = a.req.params
        lp = None
        if p.logprobs is not None:
            lp = {"token": res.token, "logprob": res.logprob, "top": res.top[:p.logprobs]}
        if a.req.constraint is not None:
            a.req.constraint.advance(res.token)
        return res.token, lp

    def _append(self, a: Active, new: List[int], lps: List[dict]) -> None:
        now = time.monotonic()
        p = a.req.params
        first = not a.generated
        out: List[int] = []
        finish = None
        for tok in new:
            a.tokens.append(tok)
            out.append(tok)
            if self.suffix is not None:
                self.suffix.push(tok)
            n_gen = len(a.tokens) - a.n_prompt
            if a.req.think is not None:
                self._think(a, tok)
            if not p.ignore_eos and n_gen >= p.min_tokens and (tok in self.cfg.eos_ids or tok in p.stop_token_ids):
                finish = Finish.STOP
                break
            if n_gen >= p.max_tokens or len(a.tokens) + 1 >= min(self.cfg.max_model_len, self.engine.max_pages_per_seq * PAGE):
                finish = Finish.LENGTH
                break
        if len(out) < len(new):
            # tokens after the stop were sampled speculatively: drop their KV
            drop = len(new) - len(out)
            a.computed = min(a.computed, len(a.tokens) - 1)
        self.stats.output_tokens += len(out)
        if first and out:
            a.t_first = now
            self.ttft.observe(now - a.req.t_submit)
        elif out and a.t_last:
            self.tpot.observe((now - a.t_last) / len(out))
        a.t_last = now
        self._emit(a, GenEvent(a.req.request_id, tokens=out, logprobs=lps or None, prompt_tokens=a.n_prompt,
                               cached_tokens=a.cached, stopped_on=out[-1] if (finish == Finish.STOP and out) else None))
        if finish is not None:
            self._retire(a, finish)

    def _think(self, a: Active, tok: int) -> None:
        th = a.req.think
        if tok == th.open_id:
            a.think_used = 0
        elif tok == th.close_id:
            a.think_used = -1
        elif a.think_used >= 0:
            a.think_used += 1
            if a.think_used >= th.budget and not a.forced:
                a.forced.extend(th.closing)
                a.think_used = -1

    def _retire(self, a: Active, why: Finish, error: Optional[str] = None, silent: bool = False) -> None:
        if a in self.active:
            self.active.remove(a)
        if self.drafter is not None and hasattr(self.drafter, "close"):
            self.drafter.close(a.req.request_id)
        if a.seq is not None:
            if why in (Finish.STOP, Finish.LENGTH) and not a.req.embed_only:
                # keep the finished conversation for follow-up turns
                n = a.seq.length - a.seq.length % PAGE
                if n >= PAGE and not self.engine.kv.gdn_layers:
                    self.cache.remember(self._key_tokens(a, n), a.seq, SnapKind.FINISH)
            self.engine.close(a.seq)
            a.seq = None
        self.stats.finished += 1
        if not silent or why != Finish.STOP:
            self._emit(a, GenEvent(a.req.request_id, finish=why, error=error, prompt_tokens=a.n_prompt,
                                   cached_tokens=a.cached))
        else:
            self._emit(a, GenEvent(a.req.request_id, finish=why, prompt_tokens=a.n_prompt, cached_tokens=a.cached))


def eng_row_index(plan, target) -> int:
    """Row index (in the step's row order) of the last row of ``target``."""
    r = 0
    for a, toks, _, _ in plan:
        r += len(toks)
        if a is target:
            return r - 1
    raise KeyError("request not in plan")
