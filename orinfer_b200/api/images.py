"""Images in chat requests: ``image_url`` content parts (data URI or http(s) URL), limits,
``detail`` and ``image_processing`` controls, UUID references with an LRU byte-budget cache,
and the binding of decoded images to placeholder runs of the tokenised prompt.

Wire format and limits follow the reference (docs/serving.md:141-174;
crates/orinfer-api/src/server/image.rs, image/cache.rs): PNG / JPEG / WebP, at most 24 MiB
compressed, 20 s fetch timeout; ``detail: "low"`` targets about 256 x 256 pixels;
``image_processing{max_pixels, max_tokens, max_tokens_per_image, max_images, auto_resize}``;
a part may carry ``"uuid"`` on first send and ``"image_url": null`` with the same uuid later;
a missing uuid is an HTTP 400 asking for the full image again.
"""

from __future__ import annotations

import base64
import binascii
import threading
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, List, Optional, Tuple

from ..models import vision as V
from .chat_codec import RequestError

MAX_IMAGE_BYTES = 24 << 20
FETCH_TIMEOUT_S = 20.0
DEFAULT_MAX_IMAGES = 20
LOW_DETAIL_PIXELS = 256 * 256
IMAGE_TEXT = "<|vision_start|><|image_pad|><|vision_end|>"


class ImageCache:
    """Decoded images by client uuid; least recently used entries go when the byte budget is
    exceeded.  A budget of 0 disables it (uuids are then never found)."""

    def __init__(self, budget_bytes: int = 256 << 20):
        self.budget = budget_bytes
        self.bytes = 0
        self._items: "OrderedDict[str, V.ImageInput]" = OrderedDict()
        self._lock = threading.Lock()

    def put(self, uuid: str, image: V.ImageInput) -> None:
        size = image.rgb.nbytes
        if size > self.budget:
            return
        with self._lock:
            old = self._items.pop(uuid, None)
            if old is not None:
                self.bytes -= old.rgb.nbytes
            self._items[uuid] = image
            self.bytes += size
            while self.bytes > self.budget:
                _, gone = self._items.popitem(last=False)
                self.bytes -= gone.rgb.nbytes

    def get(self, uuid: str) -> Optional[V.ImageInput]:
        with self._lock:
            hit = self._items.get(uuid)
            if hit is not None:
                self._items.move_to_end(uuid)
            return hit


@dataclass
class ImageOptions:
    max_pixels: Optional[int] = None
    max_tokens: Optional[int] = None
    max_tokens_per_image: Optional[int] = None
    max_images: int = DEFAULT_MAX_IMAGES
    auto_resize: bool = False

    @classmethod
    def parse(cls, value) -> "ImageOptions":
        if value is None:
            return cls()
        if not isinstance(value, dict):
            raise RequestError("`image_processing` must be an object", param="image_processing")
        unknown = set(value) - {"max_pixels", "max_tokens", "max_tokens_per_image", "max_images",
                                "auto_resize"}
        if unknown:
            raise RequestError(f"unknown image_processing field `{sorted(unknown)[0]}`",
                               param="image_processing")
        for k in ("max_pixels", "max_tokens", "max_tokens_per_image", "max_images"):
            if k in value and (not isinstance(value[k], int) or value[k] < 1):
                raise RequestError(f"`image_processing.{k}` must be a positive integer",
                                   param="image_processing")
        return cls(value.get("max_pixels"), value.get("max_tokens"),
                   value.get("max_tokens_per_image"),
                   value.get("max_images", DEFAULT_MAX_IMAGES), bool(value.get("auto_resize")))


def _fetch(url: str) -> bytes:
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if not head.endswith(";base64"):
            raise RequestError("image data URIs must be base64", param="messages")
        if len(payload) * 3 // 4 > MAX_IMAGE_BYTES:
            raise RequestError("image exceeds 24 MiB", param="messages")
        try:
            return base64.b64decode(payload, validate=True)
        except (binascii.Error, ValueError):
            raise RequestError("image data URI is not valid base64", param="messages")
    if url.startswith(("http://", "https://")):
        import requests
        try:
            with requests.get(url, stream=True, timeout=FETCH_TIMEOUT_S) as r:
                r.raise_for_status()
                data = r.raw.read(MAX_IMAGE_BYTES + 1, decode_content=True)
        except requests.RequestException as e:
            raise RequestError(f"cannot fetch image: {e}", param="messages")
        if len(data) > MAX_IMAGE_BYTES:
            raise RequestError("image exceeds 24 MiB", param="messages")
        return data
    raise RequestError("image_url must be a data URI or an http(s) URL", param="messages")


@dataclass
class BoundImages:
    prompt_ids: List[int]
    images: List[V.ImageInput] = field(default_factory=list)
    spans: List[Tuple[int, int]] = field(default_factory=list)
    rope_positions: Any = None
    rope_delta: int = 0


class ImageFrontend:
    """Everything between the JSON body and the engine for image parts."""

    def __init__(self, spec: V.VisionSpec, cache_bytes: int = 256 << 20):
        self.spec = spec
        self.cache = ImageCache(cache_bytes)

    # ---- step 1: before templating -------------------------------------------------
    def extract(self, messages: List[dict], options: ImageOptions, controls=None
                ) -> Tuple[List[dict], List[V.ImageInput]]:
        """Replace image parts by text parts holding one placeholder group each; returns the
        rewritten messages and the decoded images in prompt order.  ``controls`` maps the
        placeholder spelling to protected control-token handles (api/token_boundary.py)."""
        placeholder = controls(IMAGE_TEXT) if controls else IMAGE_TEXT
        images: List[V.ImageInput] = []
        out = []
        for mi, m in enumerate(messages):
            content = m.get("content")
            if not isinstance(content, list):
                out.append(m)
                continue
            parts = []
            for pi, part in enumerate(content):
                if not isinstance(part, dict) or part.get("type") != "image_url":
                    parts.append(part)
                    continue
                where = f"messages[{mi}].content[{pi}]"
                if len(images) >= options.max_images:
                    raise RequestError(f"more than {options.max_images} images", param=where)
                images.append(self._one(part, options, where))
                parts.append({"type": "text", "text": placeholder})
            out.append(dict(m, content=parts))
        return out, images

    def _one(self, part: dict, options: ImageOptions, where: str) -> V.ImageInput:
        ref = part.get("image_url")
        uuid = part.get("uuid") or (ref.get("uuid") if isinstance(ref, dict) else None)
        if ref is None:
            if not uuid:
                raise RequestError("image part needs `image_url` or `uuid`", param=where)
            hit = self.cache.get(str(uuid))
            if hit is None:
                raise RequestError(f"image uuid `{uuid}` is not cached; send the full image again",
                                   param=where, code="image_not_cached")
            return hit
        url = ref.get("url") if isinstance(ref, dict) else ref
        if not isinstance(url, str):
            raise RequestError("`image_url.url` must be a string", param=where)
        detail = ref.get("detail", "auto") if isinstance(ref, dict) else "auto"
        if detail not in ("auto", "low", "high"):
            raise RequestError("`detail` must be auto, low or high", param=where)
        limit = options.max_pixels
        if detail == "low":
            limit = min(limit or LOW_DETAIL_PIXELS, LOW_DETAIL_PIXELS)
        if options.max_tokens_per_image:
            per = options.max_tokens_per_image * (self.spec.patch_size * self.spec.merge_size) ** 2
            limit = min(limit or per, per)
        data = _fetch(url)
        try:
            if options.max_pixels and not options.auto_resize and detail != "low":
                # without auto_resize an oversized upload is the client's mistake, not ours to fix
                h, w = V.image_size(data)
                if h * w > options.max_pixels:
                    raise RequestError(f"image of {w}x{h} pixels exceeds `max_pixels` and "
                                       "`auto_resize` is off", param=where)
            image = V.load_image(data, self.spec, limit)
        except V.VisionError as e:
            raise RequestError(str(e), param=where)
        if uuid:
            self.cache.put(str(uuid), image)
        return image

    # ---- step 2: after tokenising ---------------------------------------------------
    def bind(self, ids: List[int], images: List[V.ImageInput], options: ImageOptions
             ) -> BoundImages:
        """Expand each single placeholder token to its image's feature count, check the span
        structure and compute the rotary positions."""
        s = self.spec
        if not images:
            if s.image_token_id in ids:
                raise RequestError("image placeholder token in a request without images",
                                   param="messages")
            return BoundImages(ids)
        counts = [V.feature_count(s, im) for im in images]
        if options.max_tokens and sum(counts) > options.max_tokens:
            raise RequestError("images exceed `image_processing.max_tokens`", param="messages")
        out, k = [], 0
        for t in ids:
            if t == s.image_token_id:
                if k >= len(images):
                    raise RequestError("more image placeholders than images", param="messages")
                out += [t] * counts[k]
                k += 1
            else:
                out.append(t)
        try:
            spans = V.image_spans(s, out, images)
        except V.VisionError as e:
            raise RequestError(str(e), param="messages")
        pos, delta = V.mrope_positions(s, out, spans,
                                       [(im.grid_height, im.grid_width) for im in images])
        return BoundImages(out, images, spans, pos, delta)


def frontend_for(tokenizer, hidden: int, cache_mib: int = 256, **spec_kw) -> ImageFrontend:
    """Frontend whose placeholder ids come from the tokenizer's vision control tokens."""
    ids = [tokenizer.token_id(t) for t in ("<|image_pad|>", "<|vision_start|>", "<|vision_end|>")]
    if any(i is None for i in ids):
        raise ValueError("the tokenizer has no vision control tokens")
    spec = V.VisionSpec(hidden=hidden, image_token_id=ids[0], vision_start_token_id=ids[1],
                        vision_end_token_id=ids[2], **spec_kw)
    return ImageFrontend(spec, cache_mib << 20)
