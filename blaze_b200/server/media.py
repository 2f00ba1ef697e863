"""Image inputs of chat requests: data URLs / local files (remote fetch is off unless allowed), size and count limits,
decode, hand-off to the vision tower.  Reference: ``crates/blaze/src/server/media.rs`` (fetch / limits / encode)."""
from __future__ import annotations

import asyncio
import base64
import io
import os
from typing import Any, Dict, List, Optional

from ..mm import ImageEmbeds, MmInput, hash_bytes
from ..service import RequestError

MAX_IMAGES = 16
MAX_IMAGE_BYTES = 20 << 20
MAX_PIXELS = 16384 * 16384


def image_bytes_of(url: str, allow_remote: bool = False, allow_files: bool = False) -> bytes:
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if ";base64" not in head:
            raise RequestError("image data URLs must be base64", "messages")
        try:
            data = base64.b64decode(payload, validate=True)
        except Exception:
            raise RequestError("image data URL is not valid base64", "messages")
    elif url.startswith("file://") and allow_files:
        path = url[7:]
        if not os.path.isfile(path):
            raise RequestError(f"image file {path!r} not found", "messages")
        with open(path, "rb") as f:
            data = f.read(MAX_IMAGE_BYTES + 1)
    elif url.startswith(("http://", "https://")):
        if not allow_remote:
            raise RequestError("remote image URLs are disabled on this server", "messages")
        import httpx
        r = httpx.get(url, timeout=10.0, follow_redirects=True)
        r.raise_for_status()
        data = r.content
    else:
        raise RequestError("unsupported image URL scheme", "messages")
    if len(data) > MAX_IMAGE_BYTES:
        raise RequestError(f"image larger than {MAX_IMAGE_BYTES >> 20} MiB", "messages")
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


def image_urls(messages: List[Dict[str, Any]]) -> List[str]:
    urls = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            for part in c:
                t = part.get("type")
                if t == "image_url":
                    u = part.get("image_url")
                    urls.append(u.get("url") if isinstance(u, dict) else u)
                elif t in ("image", "input_image") and part.get("image_url"):
                    urls.append(part["image_url"])
    return urls


async def collect_images(messages: List[Dict[str, Any]], vision, allow_remote: bool = False) -> Optional[MmInput]:
    urls = image_urls(messages)
    if not urls:
        return None
    if len(urls) > MAX_IMAGES:
        raise RequestError(f"at most {MAX_IMAGES} images per request", "messages")
    loop = asyncio.get_running_loop()

    def work():
        out = []
        for u in urls:
            data = image_bytes_of(u, allow_remote)
            img = decode_image(data)
            emb, grid = vision.encode(img)
            out.append(ImageEmbeds(emb, grid, hash_bytes(data)))
        return out
    images = await loop.run_in_executor(None, work)
    return MmInput(images, vision.image_pad_id)
