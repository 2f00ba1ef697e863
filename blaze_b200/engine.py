"""Engine: owns the model, the paged KV pools and the page allocator; runs one step at a time.

Role of the reference's ``crates/blaze/src/engine.rs``: page API ``open_from / close / snapshot /
release`` with ref-counted shared pages (:1083-1164), ``plan`` (:1168), ``step`` / ``step_sampled`` /
``prefill_only`` (:1260-1301), CUDA-graph replay keyed by step shape (``run_graph`` :326, first sight
eager, later sights captured and replayed), and a watchdog (:582-656).  Ranks here are processes
(one per GPU) that execute the same step plan; rank 0 plans and the others receive the plan over the
control group.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .batch import PAGE, SeqChunk, StepBatch, build_batch
from .config import ModelConfig
from .kv import KVCache, kv_bytes_per_token
from .models.qwen3 import Model


class OutOfPages(RuntimeError):
    pass


class DeviceStepError(RuntimeError):
    """A kernel of the step reported a failure through the device status word (a bounded wait ran out: a peer rank that
    never raised its flag, a pipeline that stalled).  The step's results are not valid; the context stays usable."""

    def __init__(self, code: int):
        names = {1: "an in-kernel barrier wait ran out", 2: "a peer rank's flag never arrived", 3: "bad kernel argument",
                 4: "a bounded device buffer overflowed"}
        super().__init__(f"device status {code}: {names.get(code, 'unknown error')}")
        self.code = code


class PageAllocator:
    """Ref-counted 16-token pages.  Page 0 is reserved as the scratch target of padded rows."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self.free: List[int] = list(range(num_pages - 1, 0, -1))
        self.refs = np.zeros(num_pages, dtype=np.int32)

    @property
    def free_count(self) -> int:
        return len(self.free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self.free):
            raise OutOfPages(f"need {n} pages, {len(self.free)} free")
        out = [self.free.pop() for _ in range(n)]
        self.refs[out] = 1
        return out

    def retain(self, pages: Sequence[int]) -> None:
        for p in pages:
            self.refs[p] += 1

    def release(self, pages: Sequence[int]) -> None:
        for p in pages:
            self.refs[p] -= 1
            if self.refs[p] == 0:
                self.free.append(p)
            elif self.refs[p] < 0:
                raise RuntimeError(f"page {p} released twice")


def make_page_allocator(num_pages: int):
    """The page allocator of the host runtime library (C++, ``csrc/runtime/repack_pages.cpp``) when that library is
    built, else the Python twin above; both have the same interface and the same allocation order."""
    import os
    if os.environ.get("BLAZE_NATIVE_PAGES", "1") != "0":
        try:
            from .runtime import NativePages
            return NativePages(num_pages)
        except Exception:
            pass
    return PageAllocator(num_pages)


@dataclass
class Seq:
    """A live sequence row: its block-table row, pages and KV length (``engine.rs:24``)."""
    row: int
    pages: List[int] = field(default_factory=list)
    length: int = 0            # tokens whose KV is in the cache
    shared: int = 0            # leading pages shared with a snapshot (never written)


@dataclass
class Snapshot:
    """A prefix-cache snapshot: shared page refs plus a recurrent-state row (``engine.rs:1119-1164``)."""
    pages: List[int]
    length: int
    state_row: int = -1


@dataclass
class EngineConfig:
    kv_tokens: int = 0                 # 0 = size from free memory
    max_seqs: int = 256
    max_model_len: int = 4096
    kv_dtype: str = "bf16"             # fp32 | bf16 | fp8
    kv_rotate: bool = False            # Hadamard-rotate q and k rows before the key is stored (fewer e4m3 outliers)
    chunk: int = 2048
    use_graphs: bool = True
    vram_reserve: int = 2 << 30
    snapshot_rows: int = 8
    hang_secs: float = 30.0
    graph_buckets: Tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)
    verify_graphs: bool = True         # chain-verify steps of equal-length chains replay captured graphs too
    verify_graph_rows: int = 1024      # ... up to this many rows per step (bucket x rows per sequence)
    feedback_eager: bool = False       # allow token feedback on uncaptured decode steps too (CPU tests of the run-ahead loop)


class Engine:
    def __init__(self, model: Model, ecfg: EngineConfig):
        self.model, self.ecfg = model, ecfg
        cfg = model.cfg
        self.device = model.device
        tpw = model.tp.world
        if cfg.has_hc and ecfg.use_graphs:
            # the stream mixing and the n-gram embedding index their state rows from the host: nothing of it is captured
            ecfg.use_graphs = False
        per_tok = max(kv_bytes_per_token(cfg, ecfg.kv_dtype, tpw), 1)
        kv_tokens = ecfg.kv_tokens
        if kv_tokens <= 0:
            if self.device.type == "cuda":
                free, _ = torch.cuda.mem_get_info(self.device)
                kv_tokens = max(int((free - ecfg.vram_reserve) // per_tok), 16 * PAGE)
                kv_tokens = min(kv_tokens, ecfg.max_seqs * ecfg.max_model_len)
            else:
                kv_tokens = min(ecfg.max_seqs * ecfg.max_model_len, 1 << 16)
        self.num_pages = kv_tokens // PAGE + 1
        self.max_pages_per_seq = (ecfg.max_model_len + PAGE - 1) // PAGE
        layout = "umma" if (self.device.type == "cuda" and ecfg.kv_dtype == "fp8" and model.ops.is_cuda) else "logical"
        if ecfg.kv_rotate and cfg.head_dim & (cfg.head_dim - 1):
            raise ValueError("kv_rotate needs a power-of-two head_dim")
        model.kv_rotate = bool(ecfg.kv_rotate)      # read by the attention prep of both op sets
        self.kv = KVCache(cfg, self.num_pages, ecfg.max_seqs, self.max_pages_per_seq, ecfg.kv_dtype, self.device,
                          layout, tpw, state_rows=ecfg.max_seqs + ecfg.snapshot_rows,
                          layers=(model.first_layer, model.last_layer))
        self.pages = make_page_allocator(self.num_pages)
        self.free_rows: List[int] = list(range(ecfg.max_seqs - 1, -1, -1))
        self.free_state_rows: List[int] = list(range(ecfg.max_seqs + ecfg.snapshot_rows - 1, ecfg.max_seqs - 1, -1))
        self.seqs: Dict[int, Seq] = {}
        self._graphs: Dict[Tuple, "_Graph"] = {}
        self._seen: Dict[Tuple, int] = {}
        self._pinned = None
        if self.device.type == "cuda":
            self._pinned = [torch.empty(1 << 19, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._pinned_ev = [None, None]
        self._pin_turn = 0
        self._last_greedy = None            # output of the last greedy decode step (source of token feedback)
        self._deferred: Dict[int, Tuple[int, int, int]] = {}   # slot -> (first row, first position, rows) of the last deferring step
        self.attn_group = 0
        if model.ops.is_cuda:
            self.attn_group = max(max(cfg.num_heads // tpw, 1) // max(cfg.num_kv_heads // tpw, 1), 1)
        # the decode attention kernel covers head_dim 128; other head sizes run every sequence through the row-block kernel
        self.attn_all_items = bool(model.ops.is_cuda and cfg.head_dim != 128)
        # Device status word, watched without a synchronisation of its own: after every step a 4-byte copy into this pinned
        # word is queued behind the step's kernels; whoever takes the step's results (and has synchronised for that)
        # calls check_status().  `status_source` replaces the device word in tests.
        self._status_host = None
        if self.device.type == "cuda" and model.ops.is_cuda:
            self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self.status_source = None
        self.status_errors = 0
        self.hangs = 0
        self._watchdog: Optional[threading.Thread] = None
        self.steps = 0
        self.last_step_started = 0.0
        self.last_step_what = ""
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.kernel_launches = 0

    # ================================================================== page API
    @property
    def free_tokens(self) -> int:
        return self.pages.free_count * PAGE

    def open_from(self, snap: Optional[Snapshot] = None) -> Seq:
        """Claim a sequence row, optionally starting from a snapshot's shared pages and state."""
        if not self.free_rows:
            raise OutOfPages("no free sequence row")
        row = self.free_rows.pop()
        s = Seq(row=row)
        if snap is not None:
            self.pages.retain(snap.pages)
            s.pages = list(snap.pages)
            s.length = snap.length
            s.shared = len(snap.pages)
            self.kv.set_pages(row, s.pages, 0)
            if snap.state_row >= 0 and self.kv.gdn_layers:
                self.kv.copy_state(snap.state_row, row)
        elif self.kv.gdn_layers:
            self.kv.zero_state(row)
        self.seqs[row] = s
        return s

    def reserve(self, s: Seq, new_len: int) -> None:
        """Make sure pages exist for positions < new_len (copy-on-write is never needed: shared
        prefixes are page-aligned and only whole pages are shared)."""
        need = (new_len + PAGE - 1) // PAGE - len(s.pages)
        if need > 0:
            if len(s.pages) + need > self.max_pages_per_seq:
                raise OutOfPages("sequence exceeds max_model_len")
            new = self.pages.alloc(need)
            self.kv.set_pages(s.row, new, len(s.pages))
            s.pages.extend(new)

    def snapshot(self, s: Seq, length: Optional[int] = None, with_state: bool = True) -> Snapshot:
        """Share the pages covering ``length`` tokens (page-aligned down) for later reuse."""
        n = s.length if length is None else min(length, s.length)
        n -= n % PAGE
        pg = s.pages[:n // PAGE]
        self.pages.retain(pg)
        row = -1
        if with_state and self.kv.gdn_layers:
            if n != s.length:
                # recurrent state is only valid at the sequence's current length
                self.pages.release(pg)
                raise ValueError("recurrent models can only snapshot at the current, page-aligned length")
            if not self.free_state_rows:
                self.pages.release(pg)
                raise OutOfPages("no free snapshot row")
            row = self.free_state_rows.pop()
            self.kv.copy_state(s.row, row)
        return Snapshot(pages=list(pg), length=n, state_row=row)

    def release(self, snap: Snapshot) -> None:
        self.pages.release(snap.pages)
        if snap.state_row >= 0:
            self.free_state_rows.append(snap.state_row)
        snap.pages = []

    def close(self, s: Seq) -> None:
        self.pages.release(s.pages)
        s.pages = []
        self.seqs.pop(s.row, None)
        self.free_rows.append(s.row)

    def truncate(self, s: Seq, length: int) -> None:
        """Drop KV beyond ``length`` (rejected speculative rows); frees whole pages no longer needed."""
        keep = (length + PAGE - 1) // PAGE
        if keep < len(s.pages):
            self.pages.release(s.pages[keep:])
            del s.pages[keep:]
        s.length = length

    # ================================================================== stepping
    def plan(self, items: Sequence[Tuple[Seq, Sequence[int], int]], defer_state: bool = False) -> List[SeqChunk]:
        """items: (seq, new tokens, rows wanting logits).  Reserves pages and advances lengths.  ``defer_state``: the rows
        are speculative — models with recurrent layers leave those sequences' state as it was, and ``commit_state`` advances
        it over the accepted rows afterwards."""
        chunks = []
        defer = bool(defer_state and self.kv.gdn_layers)
        for s, toks, want in items:
            self.reserve(s, s.length + len(toks))
            chunks.append(SeqChunk(slot=s.row, tokens=list(toks), start_pos=s.length, want_logits=want, defer_state=defer))
            s.length += len(toks)
        return chunks

    def commit_state(self, items: Sequence[Tuple[Seq, int]]) -> None:
        """items: (seq, rows kept) for sequences of the last step that ran with ``defer_state``: advance their recurrent
        state over the first ``rows kept`` rows of that step (the accepted tokens), reading the inputs the layers recorded
        (reference: ``Model::pre_verify`` / ``commit_replay``, crates/blaze/src/model.rs:3364, :3484)."""
        if not self.kv.gdn_layers or not items:
            return
        chunks, rows = [], []
        for s, keep in items:
            r0, p0, n = self._deferred[s.row]
            if keep < 1 or keep > n:
                raise ValueError("rows kept must be between 1 and the rows of the deferred step")
            chunks.append(SeqChunk(slot=s.row, tokens=[0] * keep, start_pos=p0, want_logits=0))
            rows += list(range(r0, r0 + keep))
        batch = build_batch(chunks, self.kv.block_table_host, self.device, None)
        self.h2d_bytes += batch.h2d_bytes
        self.model.gdn_replay(batch, torch.tensor(rows, dtype=torch.int32, device=self.device), self.kv)

    def plan_tree(self, items: Sequence[Tuple[Seq, Sequence[int], Sequence[int]]]) -> List[SeqChunk]:
        """items: (seq, tokens, parents) — a draft tree per sequence: ``tokens[0]`` is the last accepted token (parent -1),
        ``tokens[i]`` a drafted token whose parent row is ``parents[i] < i``.  Every row gets logits.  Row i's KV lands at
        slot ``length + i``; ``commit_tree`` moves the accepted path into place afterwards
        (reference: ``Engine::verify_many_tree``, crates/blaze/src/engine.rs :1401)."""
        if self.kv.gdn_layers:
            raise ValueError("draft trees need a model without recurrent (linear-attention) layers")
        group = max(self.model.cfg.num_heads // max(self.model.cfg.num_kv_heads, 1), 1)
        chunks = []
        for s, toks, parents in items:
            if len(toks) != len(parents) or not toks or parents[0] >= 0:
                raise ValueError("a draft tree needs one parent per token and a root with parent -1")
            if len(toks) > min(32, max(64 // group, 1)):
                raise ValueError(f"draft tree of {len(toks)} rows exceeds the verify attention's {min(32, max(64 // group, 1))}")
            self.reserve(s, s.length + len(toks))
            chunks.append(SeqChunk(slot=s.row, tokens=list(toks), start_pos=s.length, want_logits=len(toks),
                                   parents=[int(p) for p in parents]))
            s.length += len(toks)
        return chunks

    def commit_tree(self, items: Sequence[Tuple[Seq, int, Sequence[int]]]) -> None:
        """items: (seq, length before the tree step, accepted rows) — keep the root row and the accepted path (tree row
        indices, root excluded, in path order): their KV rows move to consecutive slots and the rest is dropped
        (reference: ``Engine::commit_many_tree``, crates/blaze/src/engine.rs :1478)."""
        moves = []
        for s, base, path in items:
            table = self.kv.block_table_host[s.row]
            seq_moves = []
            for k, node in enumerate(path, 1):
                if node < k:
                    raise ValueError("accepted rows must be a root-to-leaf path in row order")
                a, b = base + node, base + k
                seq_moves.append((int(table[a // PAGE]) * PAGE + a % PAGE, int(table[b // PAGE]) * PAGE + b % PAGE))
            moves.append(seq_moves)
        self.kv.move_rows(moves, self.model.ops)
        for s, base, path in items:
            self.truncate(s, base + 1 + len(path))

    def _bucket(self, rows: int) -> int:
        for b in self.ecfg.graph_buckets:
            if rows <= b:
                return b
        return rows

    def forward(self, chunks: Sequence[SeqChunk], mode: str = "greedy", hidden_in: Optional[torch.Tensor] = None,
                feedback: bool = False):
        """Run one step.  ``mode``: ``greedy`` → token ids ``[R]``; ``logits`` → fp32 ``[R, vocab]``;
        ``hidden`` → final-normed hidden rows; ``none`` → headless (prefill chunk without a head).
        ``feedback`` (captured decode steps only): the input token of row i is the token the previous captured step of
        the same bucket produced for row i, taken on the device — the caller need not have read it yet."""
        self.kv.flush()
        self.last_step_started = time.monotonic()
        self.last_step_what = f"{mode} rows={sum(len(c.tokens) for c in chunks)} seqs={len(chunks)}"
        decode_only = all(len(c.tokens) == 1 for c in chunks)
        if any(c.defer_state for c in chunks):
            self._deferred, r = {}, 0
            for c in chunks:
                if c.defer_state:
                    self._deferred[c.slot] = (r, c.start_pos, len(c.tokens))
                r += len(c.tokens)
        plain = not any(c.rope_delta or c.pos3 is not None or c.embeds for c in chunks)     # captured steps carry text rows only
        graphable = (plain and hidden_in is None and self.ecfg.use_graphs and self.device.type == "cuda" and decode_only
                     and mode == "greedy" and self.model.is_first_stage and self.model.is_last_stage and self.model.ops.is_cuda)
        # verify steps of equal-length chains (the scheduler pads drafts to one length) replay a captured graph as well
        L = len(chunks[0].tokens) if chunks else 0
        verify_graph = (not graphable and not feedback and plain and hidden_in is None and L > 1 and mode in ("greedy", "greedy_hidden")
                        and self.device.type == "cuda" and self.verify_graphable(len(chunks), L)
                        and all(len(c.tokens) == L and c.want_logits == L and c.parents is None and not c.defer_state for c in chunks))
        try:
            if graphable:
                out = self._forward_graph(chunks, feedback)
            elif verify_graph:
                out = self._forward_graph(chunks, False, L, mode)
            else:
                batch = self._build(chunks)
                if feedback:
                    if not (self.ecfg.feedback_eager and decode_only and self._last_greedy is not None):
                        raise RuntimeError("token feedback needs a captured decode step")
                    batch.tokens[:len(chunks)] = self._last_greedy[:len(chunks)].to(batch.tokens.dtype)
                out = self._run(batch, mode, hidden_in)
            if mode == "greedy" and decode_only:
                self._last_greedy = out
            if self._status_host is not None:
                self.model.ops.status_peek(self._status_host)
        finally:
            self.steps += 1
            self.last_step_started = 0.0
        return out

    def _build(self, chunks: Sequence[SeqChunk]) -> StepBatch:
        self.kv.flush()
        pinned = None
        if self._pinned is not None:
            # two staging buffers in turn: a headless prefill step is not read back by the host, so its copy may still be
            # queued when the next step is planned
            self._pin_turn ^= 1
            ev = self._pinned_ev[self._pin_turn]
            if ev is not None:
                ev.synchronize()
            pinned = self._pinned[self._pin_turn]
        batch = build_batch(chunks, self.kv.block_table_host, self.device, pinned, attn_group=self.attn_group,
                            all_items=self.attn_all_items)
        if pinned is not None:
            ev = torch.cuda.Event()
            ev.record()
            self._pinned_ev[self._pin_turn] = ev
        self.h2d_bytes += batch.h2d_bytes
        return batch

    def _run(self, batch: StepBatch, mode: str, hidden_in=None):
        hold = getattr(self.model.ops, "hold_stream", None)
        if hold is None:
            return self._run_held(batch, mode, hidden_in)
        hold()
        try:
            return self._run_held(batch, mode, hidden_in)
        finally:
            self.model.ops.release_stream()

    def _run_held(self, batch: StepBatch, mode: str, hidden_in=None):
        m = self.model
        x = m.forward(batch, self.kv, hidden_in)
        if not m.is_last_stage:
            return x
        if mode == "none":
            return None
        rows = batch.logit_rows
        if mode == "greedy":
            return m.greedy(x, rows)
        if mode == "logits":
            return m.head(x, rows)
        if mode == "hidden":
            return m.final_hidden(x, rows)
        if mode == "both":
            return m.head(x, rows), x
        if mode == "greedy_hidden":
            return m.greedy(x, rows), x
        raise ValueError(mode)

    # ------------------------------------------------------------------ CUDA graphs for decode steps
    def can_feed_back(self, n_rows: int) -> bool:
        """True when a decode step of ``n_rows`` rows would replay a captured graph (so ``feedback`` is available)."""
        if self.ecfg.feedback_eager:
            return self.model.is_first_stage and self.model.is_last_stage
        return (self.ecfg.use_graphs and self.device.type == "cuda" and self.model.ops.is_cuda and self.model.is_first_stage
                and self.model.is_last_stage and ("decode", self._bucket(n_rows)) in self._graphs)

    def verify_graphable(self, seqs: int, rows_per_seq: int) -> bool:
        """True when a step of ``seqs`` sequences with ``rows_per_seq`` rows each (chain verify) can replay a captured graph:
        the rows of one sequence must fit the decode attention kernel's row tiers and the model must keep no recurrent state."""
        from .batch import SMALL_ROWS
        return bool(self.ecfg.use_graphs and self.ecfg.verify_graphs and self.device.type == "cuda" and self.model.ops.is_cuda
                    and self.model.is_first_stage and self.model.is_last_stage and not self.kv.gdn_layers
                    and not self.attn_all_items and rows_per_seq >= 1
                    and max(self.attn_group, 1) * rows_per_seq <= SMALL_ROWS
                    and self._bucket(seqs) * rows_per_seq <= self.ecfg.verify_graph_rows)

    def _forward_graph(self, chunks: Sequence[SeqChunk], feedback: bool = False, rows_per_seq: int = 1, mode: str = "greedy"):
        B = len(chunks)
        bucket = self._bucket(B)
        key = ("decode", bucket) if rows_per_seq == 1 and mode == "greedy" else ("verify", bucket, rows_per_seq, mode)
        g = self._graphs.get(key)
        if g is None:
            seen = self._seen.get(key, 0)
            self._seen[key] = seen + 1
            if feedback:
                raise RuntimeError("token feedback needs a captured decode step")
            if seen == 0:   # first sight: run eagerly (also warms allocator and lazy inits)
                return self._run(self._build(chunks), mode)
            g = _Graph(self, bucket, rows_per_seq, mode)
            self._graphs[key] = g
        return g.replay(chunks, feedback)

    def capture_decode_graphs(self, max_batch: Optional[int] = None) -> int:
        """Capture the decode-step graph of every batch bucket up front (server start-up), so that no request pays for a
        capture.  Uses scratch sequences that are closed again; returns the number of graphs captured."""
        if not (self.ecfg.use_graphs and self.device.type == "cuda" and self.model.ops.is_cuda
                and self.model.is_first_stage and self.model.is_last_stage):
            return 0
        cap = min(max_batch or self.ecfg.max_seqs, len(self.free_rows), max(self.pages.free_count, 0))
        n = 0
        for b in self.ecfg.graph_buckets:
            if b > cap:
                break
            if ("decode", b) in self._graphs:
                continue
            seqs = [self.open_from() for _ in range(b)]
            try:
                for _ in range(2):      # first sight runs eagerly, second sight captures
                    for s in seqs:
                        s.length = 0
                    self.forward(self.plan([(s, [0], 1) for s in seqs]), "greedy")
                n += 1
            finally:
                for s in seqs:
                    self.close(s)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        return n

    def graph_kernel_count(self) -> int:
        """Kernels of this library inside one captured decode step (the largest captured bucket)."""
        return max((g.kernels for g in self._graphs.values()), default=0)

    # ================================================================== failure detection
    def check_status(self) -> None:
        """Raise ``DeviceStepError`` when a kernel of a step whose results the caller has just synchronised with reported a
        failure.  The word is cleared, so the next step starts clean (the reference fails the step's requests and keeps
        serving: ``crates/blaze/src/sched.rs:1067-1075``)."""
        if self.status_source is not None:
            code = int(self.status_source())
        elif self._status_host is not None:
            code = int(self._status_host[0])
            if code:
                self.model.ops.take_status()          # clear the device word (synchronises; this is the error path)
                self._status_host[0] = 0
        else:
            return
        if code:
            self.status_errors += 1
            raise DeviceStepError(code)

    def start_watchdog(self, on_hang=None) -> threading.Thread:
        """Report (never kill) a step that runs longer than ``hang_secs`` (``engine.rs:582-656``)."""
        if self._watchdog is not None and self._watchdog.is_alive():
            return self._watchdog

        def loop():
            while True:
                time.sleep(min(self.ecfg.hang_secs / 4, 1.0))
                t0 = self.last_step_started
                if t0 and time.monotonic() - t0 > self.ecfg.hang_secs:
                    msg = f"engine hang: step {self.steps} ({self.last_step_what}) running {time.monotonic() - t0:.1f}s"
                    self.hangs += 1
                    if on_hang:
                        on_hang(msg)
                    else:
                        from . import log
                        log.event("error", "engine.hang", what=msg)
                    self.last_step_started = 0.0
        th = threading.Thread(target=loop, name="blaze-watchdog", daemon=True)
        th.start()
        self._watchdog = th
        return th


class _Graph:
    """A captured step for a fixed sequence bucket with ``L`` rows per sequence (1 = decode, more = chain verify); inputs live
    in static buffers."""

    def __init__(self, eng: Engine, bucket: int, rows_per_seq: int = 1, mode: str = "greedy"):
        self.eng, self.bucket, self.L, self.mode = eng, bucket, rows_per_seq, mode
        dev = eng.device
        n, L = bucket, rows_per_seq
        T = n * L
        self.T = T
        self.sizes = (T, T, T, T, n, n + 1, n, T)      # tokens, positions, slot map, sequence of row, slots, q_start, ctx_len, logit rows
        self.total = sum(self.sizes)
        self.static = torch.zeros(self.total, dtype=torch.int32, device=dev)
        # two staging buffers: with token feedback the host may fill step k+1 while the copy of step k is still queued
        self.stages = [torch.zeros(self.total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.stage_ev = [None, None]      # recorded after the copy out of each stage; waited on before that stage is refilled
        self.turn = 0
        o = 0
        v = []
        self.offs = []
        for size in self.sizes:
            v.append(self.static[o:o + size])
            self.offs.append(o)
            o += size
        self.batch = StepBatch(tokens=v[0], positions=v[1], slot_mapping=v[2], seq_of_row=v[3], slots=v[4],
                               q_start=v[5], ctx_len=v[6], logit_rows=v[7], num_rows=T, max_q_len=L)
        self.batch.h_slots = [0] * n
        self.batch.h_q_start = [i * L for i in range(n + 1)]
        self.batch.h_ctx_len = [L] * n
        self.batch.h_logit_rows = list(range(T))
        self.batch.max_ctx = eng.ecfg.max_model_len
        from .batch import TINY_ROWS
        g = max(eng.attn_group, 1) * L
        if eng.attn_all_items:
            self.batch.item_seq = torch.arange(n, dtype=torch.int32, device=dev)     # one row-block item per sequence
            self.batch.item_q0 = torch.zeros(n, dtype=torch.int32, device=dev)
            self.batch.num_large = n
        elif g <= TINY_ROWS:
            self.batch.tiny_rows_max, self.batch.num_tiny = g, n
        else:
            self.batch.small_rows_max, self.batch.num_small = g, n
        self.graph = None
        self.out = None
        self.kernels = 0

    def _fill(self, chunks: Sequence[SeqChunk], feedback: bool = False) -> int:
        n, B = self.bucket, len(chunks)
        self.turn ^= 1
        stage = self.stages[self.turn]
        ev = self.stage_ev[self.turn]
        if ev is not None:
            # the copy queued from this stage two fills ago may not have run yet when the host runs far ahead of the GPU
            ev.synchronize()
        s = stage.numpy()
        bt = self.eng.kv.block_table_host
        L, T = self.L, self.T
        o_tok, o_pos, o_map, o_seq, o_slot, o_qs, o_ctx, o_lr = self.offs
        start = np.fromiter((c.start_pos for c in chunks), np.int32, B)
        slot = np.fromiter((c.slot for c in chunks), np.int32, B)
        R = B * L
        s[:] = 0
        if L == 1:
            s[o_tok:o_tok + B] = np.fromiter((c.tokens[0] for c in chunks), np.int32, B)
            pos = start
            rslot = slot
        else:
            s[o_tok:o_tok + R] = np.asarray([c.tokens for c in chunks], np.int32).reshape(-1)
            pos = (start[:, None] + np.arange(L, dtype=np.int32)[None, :]).reshape(-1)
            rslot = np.repeat(slot, L)
        s[o_pos:o_pos + R] = pos
        s[o_map:o_map + T] = -1
        s[o_map:o_map + R] = bt[rslot, pos // PAGE] * PAGE + pos % PAGE
        s[o_seq:o_seq + T] = -1
        s[o_seq:o_seq + R] = np.repeat(np.arange(B, dtype=np.int32), L) if L > 1 else np.arange(B, dtype=np.int32)
        s[o_slot:o_slot + B] = slot
        s[o_qs:o_qs + n + 1] = np.minimum(np.arange(n + 1, dtype=np.int32) * L, R)
        s[o_ctx:o_ctx + B] = start + L
        s[o_lr:o_lr + T] = np.minimum(np.arange(T, dtype=np.int32), max(R - 1, 0))
        if feedback:
            # everything but the tokens comes from the host; the tokens are the previous step's output, still on the device
            self.static[n:].copy_(stage[n:], non_blocking=True)
            self.static[:n].copy_(self.out)
            self.eng.h2d_bytes += (self.total - n) * 4
        else:
            self.static.copy_(stage, non_blocking=True)
            self.eng.h2d_bytes += self.total * 4
        ev = torch.cuda.Event()
        ev.record()
        self.stage_ev[self.turn] = ev
        return B

    def replay(self, chunks: Sequence[SeqChunk], feedback: bool = False):
        if feedback and (self.graph is None or self.L != 1):
            raise RuntimeError("token feedback needs a captured decode step")
        B = self._fill(chunks, feedback)
        if self.graph is None:
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            l0 = self.eng.model.ops.launches
            with torch.cuda.graph(self.graph):
                self.out = self.eng._run(self.batch, self.mode)
            self.kernels = self.eng.model.ops.launches - l0
        self.graph.replay()
        R = B * self.L
        if self.mode == "greedy_hidden":
            return self.out[0][:R], self.out[1][:R]
        return self.out[:R]
