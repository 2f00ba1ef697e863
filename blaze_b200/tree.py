"""Tree-verify helpers: rows of a draft tree, the accept walk, ranked alternatives
(reference: ``crates/blaze/src/tree.rs`` — ``VerifyRows``, accept walk :50, ``ranked`` :68, ``rows_of`` :82)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass
class DraftTree:
    """Node 0 is the root (the last accepted token).  ``parent[i] < i``; ``token[i]`` is the drafted token."""
    token: List[int] = field(default_factory=lambda: [-1])
    parent: List[int] = field(default_factory=lambda: [-1])

    def add(self, parent: int, token: int) -> int:
        self.token.append(token)
        self.parent.append(parent)
        return len(self.token) - 1

    def children(self, i: int) -> List[int]:
        return [j for j, p in enumerate(self.parent) if p == i]

    def depth(self, i: int) -> int:
        d = 0
        while self.parent[i] >= 0:
            i = self.parent[i]
            d += 1
        return d

    def path(self, i: int) -> List[int]:
        out = []
        while i > 0:
            out.append(i)
            i = self.parent[i]
        return out[::-1]

    def mask(self) -> List[List[bool]]:
        """mask[i][j]: row i may attend to tree row j (its ancestors and itself)."""
        n = len(self.token)
        m = [[False] * n for _ in range(n)]
        for i in range(n):
            j = i
            while j >= 0:
                m[i][j] = True
                j = self.parent[j]
        return m


def rows_of(tree: DraftTree, root_token: int) -> Tuple[List[int], List[int]]:
    """Tokens and depth offsets of the verify rows: row i feeds node i's token (root feeds ``root_token``)."""
    toks = [root_token] + tree.token[1:]
    depths = [tree.depth(i) for i in range(len(tree.token))]
    return toks, depths


def accept_walk(tree: DraftTree, chosen: Sequence[int]) -> Tuple[List[int], List[int]]:
    """``chosen[i]`` = token sampled from row i's logits.  Walk from the root: follow the child whose drafted
    token equals the parent's chosen token.  Returns (accepted node ids, emitted tokens incl. the bonus)."""
    node, path, out = 0, [], []
    while True:
        t = chosen[node]
        out.append(t)
        nxt = None
        for c in tree.children(node):
            if tree.token[c] == t:
                nxt = c
                break
        if nxt is None:
            return path, out
        path.append(nxt)
        node = nxt


def ranked(cands: Sequence[Tuple[int, float]], k: int) -> List[int]:
    """Top-k candidate ids by score, lower id first among equals."""
    return [i for i, _ in sorted(cands, key=lambda c: (-c[1], c[0]))[:k]]


def merge_chains(chains: Sequence[Sequence[int]], max_nodes: int = 32) -> DraftTree:
    """Draft tree of several candidate continuations: chains that start alike share their common rows."""
    tree = DraftTree()
    for chain in chains:
        node = 0
        for tok in chain:
            nxt = next((c for c in tree.children(node) if tree.token[c] == tok), None)
            if nxt is None:
                if len(tree.token) >= max_nodes:
                    break
                nxt = tree.add(node, int(tok))
            node = nxt
    return tree
