"""Suffix decoding: draft from earlier occurrences of the current suffix, indexed by token pairs
(reference: ``crates/blaze/src/suffix.rs`` — ``SuffixIndex`` pair-position hash, ``draft`` :105)."""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple


class SuffixIndex:
    def __init__(self, max_positions_per_pair: int = 64, max_tokens: int = 1 << 20):
        self.tokens: List[int] = []
        self.pairs: Dict[Tuple[int, int], List[int]] = {}
        self.cap, self.max_tokens = max_positions_per_pair, max_tokens

    def push(self, tok: int) -> None:
        if len(self.tokens) >= self.max_tokens:
            self.tokens, self.pairs = [], {}
        self.tokens.append(tok)
        n = len(self.tokens)
        if n >= 2:
            key = (self.tokens[-2], tok)
            lst = self.pairs.setdefault(key, [])
            lst.append(n - 1)           # position of the pair's second token
            if len(lst) > self.cap:
                del lst[0]

    def extend(self, toks: Sequence[int]) -> None:
        for t in toks:
            self.push(t)

    def draft(self, history: Sequence[int], k: int, min_match: int = 2) -> List[int]:
        """Best continuation: the occurrence with the longest matching context; ties → most recent."""
        if len(history) < 2 or k <= 0:
            return []
        key = (history[-2], history[-1])
        best_len, best_pos = 0, -1
        for pos in reversed(self.pairs.get(key, [])):
            if pos + 1 >= len(self.tokens):
                continue
            m = 2
            while m < 32 and pos - m >= 0 and m < len(history) and self.tokens[pos - m] == history[-1 - m]:
                m += 1
            if m > best_len:
                best_len, best_pos = m, pos
        if best_pos < 0 or best_len < min_match:
            return []
        return self.tokens[best_pos + 1:best_pos + 1 + k]

    def score(self, history: Sequence[int], k: int) -> Tuple[List[int], float]:
        """Draft plus a confidence in [0, 1] growing with the matched context length."""
        d = self.draft(history, k)
        if not d:
            return [], 0.0
        return d, min(1.0, 0.25 + 0.1 * len(d))
