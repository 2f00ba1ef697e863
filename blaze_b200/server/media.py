"""Image inputs of chat requests: data URLs / local files (remote fetch is off unless allowed), size and count limits,
decode, hand-off to the vision tower.  Reference: ``crates/blaze/src/server/media.rs`` (fetch / limits / encode)."""
from __future__ import annotations

import asyncio
import base64
import io
import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple
from urllib.parse import urlparse

from ..mm import ImageEmbeds, MmInput, hash_bytes
from ..service import RequestError

MAX_PIXELS = 16384 * 16384


def parse_limit(text: Optional[str]) -> int:
    """``--limit-mm-per-prompt``: most images of one request, as JSON (``{"image": 4}`` or ``{"image": {"count": 4}}``) or
    ``image=4``; anything that does not mention images leaves the default of 999."""
    s = (text or "").strip()
    if not s:
        return 999
    if s.startswith("{"):
        try:
            v = json.loads(s)
        except ValueError as e:
            raise ValueError(f"--limit-mm-per-prompt: {e}")
        x = v.get("image") if isinstance(v, dict) else None
        if x is None:
            return 999
        n = x.get("count") if isinstance(x, dict) else x
        if isinstance(n, bool) or not isinstance(n, int) or n < 0:
            raise ValueError("--limit-mm-per-prompt: image needs a count")
        return n
    for pair in s.split(","):
        k, _, v = pair.partition("=")
        if k.strip() == "image":
            try:
                return int(v.strip())
            except ValueError:
                raise ValueError(f"--limit-mm-per-prompt: bad count {v.strip()!r}")
    return 999


@dataclass
class MediaPolicy:
    """What image input a server accepts (``crates/blaze/src/server/media.rs`` ``MmConfig``; flags of ``main.rs:484-511``)."""
    limit_images: int = 999                       # --limit-mm-per-prompt
    low_detail_pixels: int = 512 * 512            # --mm-low-detail-pixels: max_pixels of image_url.detail "low" (0 ignores detail)
    fetch_timeout_s: float = 5.0                  # --image-fetch-timeout: all http(s) downloads of one request together
    fetch_max_bytes: int = 64 << 20               # --image-fetch-max-mib
    allowed_domains: Tuple[str, ...] = ()         # --allowed-media-domains (empty: any host)
    processor: Dict[str, Any] = field(default_factory=dict)     # --mm-processor-kwargs: min_pixels, max_pixels, size.{shortest,longest}_edge
    enabled: bool = True                          # --vision off

    def pixel_limits(self, cfg, overrides: Optional[Dict[str, Any]] = None, detail: Optional[str] = None) -> Tuple[int, int]:
        """(min_pixels, max_pixels) of one image: the checkpoint's processor settings, then the server's, then the
        request's ``mm_processor_kwargs``, then the cap of ``detail: "low"``."""
        lo, hi = int(cfg.min_pixels), int(cfg.max_pixels)
        for src, what in ((self.processor, "--mm-processor-kwargs"), (overrides or {}, "mm_processor_kwargs")):
            if not isinstance(src, dict):
                raise RequestError(f"{what} must be an object", "mm_processor_kwargs")
            size = src.get("size") if isinstance(src.get("size"), dict) else {}
            for key, alt in (("min_pixels", "shortest_edge"), ("max_pixels", "longest_edge")):
                v = src.get(key, size.get(alt))
                if v is None:
                    continue
                if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                    raise RequestError(f"{what}.{key} must be a positive integer", "mm_processor_kwargs")
                if key == "min_pixels":
                    lo = v
                else:
                    hi = v
        if lo > hi:
            raise RequestError(f"min_pixels {lo} is above max_pixels {hi}", "mm_processor_kwargs")
        if detail is not None:
            if detail not in ("auto", "high", "low"):
                raise RequestError(f"image_url.detail must be auto, low or high, not {detail!r}", "messages")
            if detail == "low" and self.low_detail_pixels > 0:
                hi = min(hi, self.low_detail_pixels)
                lo = min(lo, hi)
        return lo, hi

    def host_allowed(self, url: str) -> None:
        host = (urlparse(url).hostname or "").lower()
        if self.allowed_domains and not any(host == d or host.endswith("." + d) for d in self.allowed_domains):
            raise RequestError(f"the URL's domain {host!r} is not allowed: allowed domains are {list(self.allowed_domains)}", "messages")


def image_bytes_of(url: str, allow_remote: bool = False, allow_files: bool = False, policy: Optional[MediaPolicy] = None,
                   deadline: Optional[float] = None, fetch=None) -> bytes:
    """The bytes behind an image URL: a base64 ``data:`` URL, or an http(s) URL when remote fetch is allowed (within the
    policy's domains, size and time limits; ``fetch(url, timeout)`` is the download call, ``httpx.get`` by default)."""
    policy = policy or MediaPolicy()
    limit = policy.fetch_max_bytes
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if ";base64" not in head:
            raise RequestError("data URLs of images must be base64", "messages")
        try:
            data = base64.b64decode(payload, validate=True)
        except Exception:
            raise RequestError("image data URL is not valid base64", "messages")
    elif url.startswith("file://") and allow_files:
        path = url[7:]
        if not os.path.isfile(path):
            raise RequestError(f"image file {path!r} not found", "messages")
        with open(path, "rb") as f:
            data = f.read(limit + 1)
    elif url.startswith(("http://", "https://")):
        if not allow_remote:
            raise RequestError("remote image URLs are disabled on this server", "messages")
        policy.host_allowed(url)
        left = policy.fetch_timeout_s if deadline is None else deadline - time.monotonic()
        if left <= 0:
            raise RequestError("the request's image downloads took longer than their time limit", "messages")
        if fetch is None:
            import httpx

            def fetch(u, timeout):
                r = httpx.get(u, timeout=timeout, follow_redirects=True)
                r.raise_for_status()
                return r.content
        try:
            data = fetch(url, left)
        except RequestError:
            raise
        except Exception as e:
            raise RequestError(f"cannot fetch the image: {e}", "messages")
    else:
        raise RequestError("the image URL must be a data: URL (base64) or an http(s) URL", "messages")
    if len(data) > limit:
        raise RequestError(f"the image is larger than the limit of {limit} bytes", "messages")
    return data


def decode_image(data: bytes):
    from PIL import Image
    try:
        img = Image.open(io.BytesIO(data))
        img.load()
    except Exception:
        raise RequestError("image could not be decoded", "messages")
    if img.width * img.height > MAX_PIXELS:
        raise RequestError("image has too many pixels", "messages")
    return img.convert("RGB")


def image_parts(messages: List[Dict[str, Any]]) -> List[Tuple[str, Optional[str]]]:
    """The image content parts of the messages in prompt order: (url, detail).  Other media are refused here."""
    out: List[Tuple[str, Optional[str]]] = []
    for m in messages:
        c = m.get("content") if isinstance(m, dict) else None
        if not isinstance(c, list):
            continue
        for part in c:
            if not isinstance(part, dict):
                continue
            t = part.get("type")
            if t in ("image_url", "image", "input_image"):
                src = part.get("image_url", part.get("image"))
                if isinstance(src, dict):
                    url, detail = src.get("url"), src.get("detail", part.get("detail"))
                else:
                    url, detail = src, part.get("detail")
                if not isinstance(url, str) or not url:
                    raise RequestError("an image part needs image_url.url", "messages")
                out.append((url, detail if isinstance(detail, str) else None))
            elif t in ("video_url", "video", "audio_url", "input_audio", "audio"):
                raise RequestError(f"content part {t!r} is not supported: this server reads images only", "messages")
    return out


def image_urls(messages: List[Dict[str, Any]]) -> List[str]:
    return [u for u, _ in image_parts(messages)]


async def collect_images(messages: List[Dict[str, Any]], vision, allow_remote: bool = False, policy: Optional[MediaPolicy] = None,
                         overrides: Optional[Dict[str, Any]] = None, fetch=None) -> Optional[MmInput]:
    """Load, decode and encode the request's images (off the event loop).  ``overrides``: the request's
    ``mm_processor_kwargs``."""
    policy = policy or MediaPolicy()
    parts = image_parts(messages)
    if not parts:
        return None
    if vision is None or not policy.enabled:
        raise RequestError("this server takes no image input (it was started with --vision off, or the model has no vision tower)",
                           "messages")
    if len(parts) > policy.limit_images:
        raise RequestError(f"At most {policy.limit_images} image(s) may be provided in one prompt.", "messages")
    limits = [policy.pixel_limits(vision.cfg, overrides, d) for _, d in parts]       # validates before any download
    loop = asyncio.get_running_loop()
    deadline = time.monotonic() + policy.fetch_timeout_s

    def work():
        out = []
        for (u, _), (lo, hi) in zip(parts, limits):
            data = image_bytes_of(u, allow_remote, policy=policy, deadline=deadline, fetch=fetch)
            img = decode_image(data)
            emb, grid = vision.encode(img, min_pixels=lo, max_pixels=hi)
            out.append(ImageEmbeds(emb, grid, hash_bytes(data + f"|{lo}|{hi}".encode())))
        return out
    images = await loop.run_in_executor(None, work)
    return MmInput(images, vision.image_pad_id)
