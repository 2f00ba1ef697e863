"""Non-zero ranks of a served model: execute the step plans that rank 0 broadcasts.

The reference's ranks are threads fed through channels (``Cmd`` / ``Reply`` in ``crates/blaze/src/engine.rs:94-166``,
``broadcast`` :1042).  Here ranks are processes: rank 0's engine publishes each step (page reservations + chunks + mode)
over the control group, the followers replay it on their engine so that every rank launches the same kernels in the
same order.
"""
from __future__ import annotations

from typing import List, Tuple

from ..batch import SeqChunk


class Leader:
    """Wraps rank 0's engine so that every ``forward`` is mirrored on the followers.  ``tag`` names the engine on the
    followers' side: 0 = the served model, 1 = the drafter's one-layer model (cut over the ranks like the target, so its
    steps run the same collectives and must be launched on every rank)."""

    def __init__(self, engine, group, tag: int = 0):
        self.engine, self.group, self.tag = engine, group, tag
        self._forward = engine.forward
        self._sent = {}          # row -> page list as the followers know it
        engine.forward = self.forward
        ct, cs = engine.commit_tree, engine.commit_state

        def commit_tree(items):
            self.call("commit_tree", [(s.row, base, list(path)) for s, base, path in items])
            return ct(items)

        def commit_state(items):
            if engine.kv.gdn_layers and items:
                self.call("commit_state", [(s.row, keep) for s, keep in items])
            return cs(items)
        engine.commit_tree, engine.commit_state = commit_tree, commit_state

    def forward(self, chunks, mode="greedy", hidden_in=None, feedback=False):
        # only the rows whose page list changed since the last step travel (a decode step changes one row in sixteen)
        changed, live = {}, self.engine.seqs
        for r, s in live.items():
            old = self._sent.get(r)
            if old is None or len(old) != len(s.pages) or old != s.pages:
                changed[r] = list(s.pages)
                self._sent[r] = changed[r]
        gone = [r for r in self._sent if r not in live]
        for r in gone:
            del self._sent[r]
        hid = None if hidden_in is None else (tuple(hidden_in.shape), str(hidden_in.dtype).replace("torch.", ""))
        plan = ("step", mode, [(c.slot, list(c.tokens), c.start_pos, c.want_logits, c.parents, c.defer_state) for c in chunks],
                changed, gone, feedback, self.tag, hid)
        self.group.broadcast_object(plan, 0)
        if hidden_in is not None:
            # input rows that only rank 0 has computed (the drafter's fused embedding + hidden rows) follow the plan
            hidden_in = hidden_in.contiguous()
            self.group.broadcast(hidden_in, 0)
        return self._forward(chunks, mode, hidden_in, feedback)

    def call(self, method: str, *args):
        """Mirror an engine call that is not a step (KV row moves after a tree step, replay of deferred recurrent state)."""
        self.group.broadcast_object(("call", method, args), 0)

    def quit(self):
        self.group.broadcast_object(("quit",), 0)


def follow(llm) -> int:
    """Follower loop: mirror rank 0's sequence table and run the same steps."""
    import torch
    engines = {0: llm.engine}
    drafter = getattr(llm, "drafter", None)
    if drafter is not None and hasattr(drafter, "engine"):
        engines[1] = drafter.engine
    group = getattr(llm, "group", None) or llm.model.tp.group
    from ..engine import Seq
    while True:
        eng = engines[0]
        msg = group.broadcast_object(None, 0)
        if msg[0] == "quit":
            return 0
        if msg[0] == "call":
            _, method, args = msg
            if method == "commit_tree":
                eng.commit_tree([(eng.seqs[row], base, path) for row, base, path in args[0]])
            elif method == "commit_state":
                eng.commit_state([(eng.seqs[row], keep) for row, keep in args[0]])
            continue
        _, mode, raw, changed, gone, feedback, tag, hid = msg
        eng = engines[tag]
        hidden_in = None
        if hid is not None:
            hidden_in = torch.empty(hid[0], dtype=getattr(torch, hid[1]), device=eng.device)
            group.broadcast(hidden_in, 0)
        # mirror the page tables (same allocator decisions are implied by copying rank 0's)
        for row, pg in changed.items():
            s = eng.seqs.get(row)
            if s is None:
                s = Seq(row=row)
                eng.seqs[row] = s
            if pg != s.pages:
                keep = 0
                while keep < min(len(pg), len(s.pages)) and pg[keep] == s.pages[keep]:
                    keep += 1
                eng.kv.set_pages(row, pg[keep:], keep)
                s.pages = list(pg)
        for row in gone:
            eng.seqs.pop(row, None)
        chunks = [SeqChunk(slot, toks, start, want, parents=parents, defer_state=defer) for slot, toks, start, want, parents, defer in raw]
        for c in chunks:                      # the follower's sequence lengths follow the plan (tree commits read them)
            s = eng.seqs.get(c.slot)
            if s is not None:
                s.length = c.start_pos + len(c.tokens)
        eng.forward(chunks, mode, hidden_in=hidden_in, feedback=feedback)


def attach(llm, group, pp_chunk: int = 512):
    """Connect one rank's engine to the others: pipeline stages first (``engine.forward`` then runs this stage's part of
    a step), then the step protocol — global rank 0 gets a :class:`Leader` and returns it, every other rank should call
    :func:`follow`."""
    if group is None:
        return None
    if getattr(group, "stages", 1) > 1:
        from .pp import Pipeline
        llm.pipeline = Pipeline(llm.engine, group, pp_chunk)
    if group.global_rank == 0:
        llm.leader = Leader(llm.engine, group)
        drafter = getattr(llm, "drafter", None)
        if drafter is not None and hasattr(drafter, "engine") and group.world > 1:
            if getattr(drafter, "kind", "mtp") != "mtp":
                # their passes do not go through the drafter engine's forward yet, so the followers would not run them
                raise RuntimeError(f"the {drafter.kind} drafter is not available with tensor-parallel follower ranks; use --spec-method mtp")
            llm.draft_leader = Leader(drafter.engine, group, tag=1)
        return llm.leader
    return None
