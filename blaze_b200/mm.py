"""Multimodal inputs: image embeddings spliced into the token stream, 3-axis (M-RoPE) positions, prefix-cache keys.

Reference: ``crates/blaze/src/mm.rs`` — ``ImageEmbeds``, ``MmInput`` 3-axis positions :64, ``segments`` :89, cache keys
>= 1<<62 derived from a keyed hash of the image bytes :102-122 (blake3 there and here).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

CACHE_KEY_BASE = 1 << 62


def hash_bytes(data: bytes, key: bytes = b"blaze-image-key".ljust(32, b"\0")) -> int:
    """Keyed content hash folded into the prefix-cache key space (ids >= 2^62 never collide with token ids)."""
    try:
        import blake3
        d = blake3.blake3(data, key=key).digest()
    except ImportError:  # pragma: no cover
        import hashlib
        d = hashlib.blake2b(data, key=key[:32], digest_size=32).digest()
    return CACHE_KEY_BASE | (int.from_bytes(d[:8], "little") & (CACHE_KEY_BASE - 1))


@dataclass
class ImageEmbeds:
    embeds: torch.Tensor          # [n_tokens, hidden] output of the vision tower (after the merger)
    grid: Tuple[int, int]         # merged (h, w) token grid
    key: int                      # content hash (cache key)


@dataclass
class MmInput:
    images: List[ImageEmbeds] = field(default_factory=list)
    image_pad_id: int = -1

    def segments(self, tokens: Sequence[int]) -> List[Tuple[int, int, int]]:
        """(start, end, image index) of each run of image-pad tokens, in order."""
        out, i, k = [], 0, 0
        while i < len(tokens):
            if tokens[i] == self.image_pad_id:
                j = i
                while j < len(tokens) and tokens[j] == self.image_pad_id:
                    j += 1
                out.append((i, j, k))
                k += 1
                i = j
            else:
                i += 1
        return out

    def expand(self, tokens: Sequence[int]) -> List[int]:
        """Replace each single image-pad placeholder by as many pads as its image has tokens."""
        out: List[int] = []
        k = 0
        for t in tokens:
            if t == self.image_pad_id and k < len(self.images):
                out.extend([t] * self.images[k].embeds.shape[0])
                k += 1
            else:
                out.append(t)
        return out

    def positions3(self, tokens: Sequence[int]) -> torch.Tensor:
        """M-RoPE positions ``[3, T]`` (temporal, height, width): text advances all three axes together; an image block
        keeps t fixed and spreads h / w over its grid; text after it resumes from the block's largest position + 1."""
        T = len(tokens)
        pos = torch.zeros(3, T, dtype=torch.int32)
        nxt, i = 0, 0
        segs = {s: (e, k) for s, e, k in self.segments(tokens)}
        while i < T:
            if i in segs:
                e, k = segs[i]
                h, w = self.images[k].grid if k < len(self.images) else (1, e - i)
                n = e - i
                idx = torch.arange(n)
                pos[0, i:e] = nxt
                pos[1, i:e] = nxt + (idx // max(w, 1)).to(torch.int32)
                pos[2, i:e] = nxt + (idx % max(w, 1)).to(torch.int32)
                nxt += max(h, w)
                i = e
            else:
                pos[:, i] = nxt
                nxt += 1
                i += 1
        return pos

    def cache_tokens(self, tokens: Sequence[int]) -> List[int]:
        """Token list for prefix-cache matching: image pads are replaced by the image's content key."""
        out = list(tokens)
        for s, e, k in self.segments(tokens):
            if k < len(self.images):
                for j in range(s, e):
                    out[j] = self.images[k].key
        return out

    def splice(self, tokens: Sequence[int], embeds: torch.Tensor, row0: int = 0) -> torch.Tensor:
        """Overwrite the embedding rows of image-pad positions with the tower's outputs.  ``embeds`` holds rows
        ``row0 .. row0 + len(embeds)`` of the sequence."""
        for s, e, k in self.segments(tokens):
            if k >= len(self.images):
                continue
            lo, hi = max(s, row0), min(e, row0 + embeds.shape[0])
            if lo < hi:
                embeds[lo - row0:hi - row0] = self.images[k].embeds[lo - s:hi - s].to(embeds.dtype)
        return embeds
