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
    """Wraps rank 0's engine so that every ``forward`` is mirrored on the followers."""

    def __init__(self, engine, group):
        self.engine, self.group = engine, group
        self._forward = engine.forward
        self._sent = {}          # row -> page list as the followers know it
        engine.forward = self.forward

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
        plan = ("step", mode, [(c.slot, list(c.tokens), c.start_pos, c.want_logits) for c in chunks], changed, gone, feedback)
        self.group.broadcast_object(plan, 0)
        return self._forward(chunks, mode, hidden_in, feedback)

    def quit(self):
        self.group.broadcast_object(("quit",), 0)


def follow(llm) -> int:
    """Follower loop: mirror rank 0's sequence table and run the same steps."""
    eng, group = llm.engine, llm.model.tp.group
    from ..engine import Seq
    while True:
        msg = group.broadcast_object(None, 0)
        if msg[0] == "quit":
            return 0
        _, mode, raw, changed, gone, feedback = msg
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
        chunks = [SeqChunk(slot, toks, start, want) for slot, toks, start, want in raw]
        eng.forward(chunks, mode, feedback=feedback)
