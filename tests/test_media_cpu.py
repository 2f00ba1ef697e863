"""Image input policy of the server (``blaze_b200/server/media.py``): count limit, ``detail``, processor overrides, domains,
download limits, refusal of other media and of servers without a tower (reference: ``crates/blaze/src/server/media.rs``)."""
import asyncio
import base64
import io

import pytest
import torch

from blaze_b200.models.vision import Vision, VisionConfig, VisionTower
from blaze_b200.server.media import MediaPolicy, collect_images, image_parts, parse_limit
from blaze_b200.service import RequestError


def _png(w=64, h=48, seed=0):
    from PIL import Image
    g = torch.Generator().manual_seed(seed)
    arr = (torch.rand(h, w, 3, generator=g) * 255).to(torch.uint8).numpy()
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    return buf.getvalue()


def _data_url(data):
    return "data:image/png;base64," + base64.b64encode(data).decode()


@pytest.fixture(scope="module")
def vision():
    cfg = VisionConfig(hidden_size=64, num_heads=2, intermediate_size=128, depth=1, out_hidden_size=64, num_position_embeddings=64)
    return Vision(VisionTower.random_init(cfg, "cpu"), image_pad_id=300)


def _msgs(*parts):
    return [{"role": "user", "content": [{"type": "text", "text": "look"}, *parts]}]


def _run(coro):
    return asyncio.run(coro)


def test_limit_flag_forms():
    assert parse_limit("") == 999 and parse_limit("image=3") == 3 and parse_limit('{"image": 2}') == 2
    assert parse_limit('{"image": {"count": 5}}') == 5 and parse_limit('{"video": 1}') == 999 and parse_limit("video=2") == 999
    for bad in ("image=many", '{"image": "x"}', "{not json"):
        with pytest.raises(ValueError):
            parse_limit(bad)


def test_parts_detail_and_other_media():
    parts = image_parts(_msgs({"type": "image_url", "image_url": {"url": "u1", "detail": "low"}},
                              {"type": "image_url", "image_url": "u2"}, {"type": "input_image", "image_url": "u3", "detail": "high"}))
    assert parts == [("u1", "low"), ("u2", None), ("u3", "high")]
    with pytest.raises(RequestError, match="images only"):
        image_parts(_msgs({"type": "video_url", "video_url": {"url": "v"}}))
    with pytest.raises(RequestError, match="image_url.url"):
        image_parts(_msgs({"type": "image_url", "image_url": {}}))


def test_pixel_limits_layers(vision):
    pol = MediaPolicy(processor={"max_pixels": 200 * 200}, low_detail_pixels=100 * 100)
    cfg = vision.cfg
    assert pol.pixel_limits(cfg) == (cfg.min_pixels, 200 * 200)
    assert pol.pixel_limits(cfg, {"size": {"longest_edge": 150 * 150}}) == (cfg.min_pixels, 150 * 150)      # the request wins
    assert pol.pixel_limits(cfg, None, "low") == (cfg.min_pixels, 100 * 100) and pol.pixel_limits(cfg, None, "high")[1] == 200 * 200
    assert MediaPolicy(low_detail_pixels=0).pixel_limits(cfg, None, "low")[1] == cfg.max_pixels                # 0 ignores detail
    with pytest.raises(RequestError, match="above max_pixels"):
        pol.pixel_limits(cfg, {"min_pixels": 300 * 300})
    with pytest.raises(RequestError, match="auto, low or high"):
        pol.pixel_limits(cfg, None, "ultra")
    with pytest.raises(RequestError, match="positive integer"):
        pol.pixel_limits(cfg, {"max_pixels": -1})


def test_collect_images_policy(vision):
    img = _data_url(_png())
    mm = _run(collect_images(_msgs({"type": "image_url", "image_url": {"url": img}}), vision))
    assert len(mm.images) == 1 and mm.images[0].embeds.shape[1] == 64
    # detail "low" caps the pixels: fewer image tokens than the same picture at the processor's own limits
    big = _data_url(_png(448, 448, 1))
    full = _run(collect_images(_msgs({"type": "image_url", "image_url": {"url": big}}), vision, policy=MediaPolicy(low_detail_pixels=112 * 112)))
    low = _run(collect_images(_msgs({"type": "image_url", "image_url": {"url": big, "detail": "low"}}), vision,
                              policy=MediaPolicy(low_detail_pixels=112 * 112)))
    assert low.images[0].embeds.shape[0] < full.images[0].embeds.shape[0]
    assert low.images[0].key != full.images[0].key                       # different pixels, different cache key
    assert _run(collect_images([{"role": "user", "content": "no images"}], vision)) is None
    two = _msgs({"type": "image_url", "image_url": {"url": img}}, {"type": "image_url", "image_url": {"url": img}})
    with pytest.raises(RequestError, match="At most 1 image"):
        _run(collect_images(two, vision, policy=MediaPolicy(limit_images=1)))
    with pytest.raises(RequestError, match="no image input"):
        _run(collect_images(two, vision, policy=MediaPolicy(enabled=False)))
    with pytest.raises(RequestError, match="no image input"):
        _run(collect_images(two, None))
    with pytest.raises(RequestError, match="must be base64"):
        _run(collect_images(_msgs({"type": "image_url", "image_url": {"url": "data:image/png,abc"}}), vision))


def test_remote_images_domains_size_and_time(vision):
    data = _png()
    calls = []

    def fetch(url, timeout):
        calls.append((url, timeout))
        return data

    msgs = _msgs({"type": "image_url", "image_url": {"url": "https://img.example.com/a.png"}})
    with pytest.raises(RequestError, match="disabled"):
        _run(collect_images(msgs, vision, allow_remote=False, fetch=fetch))
    mm = _run(collect_images(msgs, vision, allow_remote=True, policy=MediaPolicy(allowed_domains=("example.com",)), fetch=fetch))
    assert len(mm.images) == 1 and calls and 0 < calls[0][1] <= 5.0
    with pytest.raises(RequestError, match="not allowed"):
        _run(collect_images(msgs, vision, allow_remote=True, policy=MediaPolicy(allowed_domains=("other.org",)), fetch=fetch))
    with pytest.raises(RequestError, match="larger than the limit"):
        _run(collect_images(msgs, vision, allow_remote=True, policy=MediaPolicy(fetch_max_bytes=100), fetch=fetch))
    with pytest.raises(RequestError, match="time limit"):
        _run(collect_images(msgs, vision, allow_remote=True, policy=MediaPolicy(fetch_timeout_s=0.0), fetch=fetch))

    def broken(url, timeout):
        raise OSError("connection refused")
    with pytest.raises(RequestError, match="cannot fetch"):
        _run(collect_images(msgs, vision, allow_remote=True, fetch=broken))
    with pytest.raises(RequestError, match="data: URL"):
        _run(collect_images(_msgs({"type": "image_url", "image_url": {"url": "ftp://x/y.png"}}), vision, allow_remote=True))


def test_service_flags_reach_the_policy():
    from blaze_b200.cli import build_parser
    from blaze_b200.server.run import service_args_of
    ns = build_parser().parse_args(["serve", "--model", "tiny", "--limit-mm-per-prompt", "image=2", "--mm-low-detail-pixels", "1024",
                                    "--image-fetch-timeout", "2.5", "--image-fetch-max-mib", "8", "--allowed-media-domains", "a.com, B.org",
                                    "--mm-processor-kwargs", '{"max_pixels": 4096}', "--vision", "cpu", "--vision-threads", "3",
                                    "--thinking-budget", "256", "--temperature", "0.6", "--top-k", "20", "--max-tokens", "99"])
    svc = service_args_of(ns)
    assert svc.limit_mm_per_prompt == 2 and svc.mm_low_detail_pixels == 1024 and svc.image_fetch_timeout == 2.5
    assert svc.image_fetch_max_mib == 8 and svc.allowed_media_domains == ("a.com", "b.org") and svc.mm_processor_kwargs == {"max_pixels": 4096}
    assert svc.vision == "cpu" and svc.vision_threads == 3 and svc.thinking_budget == 256
    assert svc.defaults["temperature"] == 0.6 and svc.defaults["top_k"] == 20 and svc.default_max_tokens == 99
    with pytest.raises(SystemExit):
        service_args_of(build_parser().parse_args(["serve", "--model", "tiny", "--limit-mm-per-prompt", "image=x"]))
