"""Image inputs for the decoder: geometry, patch packing, span binding, MRoPE positions, the
ViT-style encoder whose features overlay the image placeholder rows, and the feature cache.

Contracts follow the reference's crates/orinfer-model-sdk/src/vision.rs (``VisionSpec``:
patch 16, temporal patch 2, 2x2 merger; ``grid_features``; ``feature_count``; ``image_spans``
binding media to complete placeholder runs; checkpoint patch order merge-block / patch /
channel / temporal / spatial with ``rgb / 127.5 - 1``), crates/orinfer-engine/src/vision/
pixels.rs + features.rs (exact packing, model-scoped feature cache keyed independently of token
positions) and its interleaved MRoPE rule (sections 11/11/10 of 32 frequencies,
kernels/cuda/model/kv_int8.py:63-206).  The encoder itself is plain PyTorch (fp16 on the GPU):
it runs once per distinct image and is not on the token-rate path.
"""

from __future__ import annotations

import hashlib
import io
import math
from collections import OrderedDict
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


class VisionError(ValueError):
    pass


@dataclass
class VisionSpec:
    hidden: int                      # decoder hidden size (feature width)
    image_token_id: int
    vision_start_token_id: int
    vision_end_token_id: int
    patch_size: int = 16
    temporal_patch_size: int = 2
    merge_size: int = 2
    max_patches: int = 16384
    max_features: int = 4096
    min_pixels: int = 256 * 256
    max_pixels: int = 1024 * 1024
    width: int = 128                 # encoder width
    depth: int = 2
    heads: int = 4

    @property
    def patch_values(self) -> int:
        return self.patch_size * self.patch_size * self.temporal_patch_size * 3

    def grid_features(self, height: int, width: int) -> int:
        patches = height * width
        if height <= 0 or width <= 0 or patches > self.max_patches:
            raise VisionError("invalid image grid or vision capacity")
        if height % self.merge_size or width % self.merge_size:
            raise VisionError("image grid must align to the merger")
        return patches // (self.merge_size * self.merge_size)


@dataclass
class ImageInput:
    grid_height: int                 # in patches
    grid_width: int
    rgb: np.ndarray                  # uint8 [grid_height * patch, grid_width * patch, 3]

    def digest(self) -> int:
        h = hashlib.sha256()
        h.update(f"{self.grid_height}x{self.grid_width}:".encode())
        h.update(np.ascontiguousarray(self.rgb).tobytes())
        return int.from_bytes(h.digest()[:8], "little")


def feature_count(spec: VisionSpec, image: ImageInput) -> int:
    n = spec.grid_features(image.grid_height, image.grid_width)
    want = (image.grid_height * spec.patch_size, image.grid_width * spec.patch_size, 3)
    if tuple(image.rgb.shape) != want or image.rgb.dtype != np.uint8:
        raise VisionError("invalid image grid, pixel data or vision capacity")
    return n


def image_spans(spec: VisionSpec, tokens: Sequence[int], images: Sequence[ImageInput]
                ) -> List[Tuple[int, int]]:
    """Bind every image to one complete run of placeholder tokens, in order: [(start, end)].
    Missing markers, short runs, stray placeholders and feature overflow are errors."""
    spans, cursor, total = [], 0, 0
    toks = list(tokens)
    for image in images:
        try:
            start = toks.index(spec.image_token_id, cursor)
        except ValueError:
            raise VisionError("image marker missing") from None
        n = feature_count(spec, image)
        total += n
        if total > spec.max_features:
            raise VisionError("image feature capacity exceeded")
        cursor = start + n
        if cursor > len(toks):
            raise VisionError("image span outside prompt")
        if any(t != spec.image_token_id for t in toks[start:cursor]):
            raise VisionError("invalid image token span")
        spans.append((start, cursor))
    if spec.image_token_id in toks[cursor:]:
        raise VisionError("unbound image tokens")
    return spans


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int
                 ) -> Tuple[int, int]:
    """Target size: both sides multiples of ``factor`` (patch x merge), area inside
    [min_pixels, max_pixels], aspect ratio kept as far as rounding allows."""
    if height <= 0 or width <= 0 or max(height, width) / min(height, width) > 200:
        raise VisionError("unsupported image aspect ratio")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def image_size(data: bytes) -> Tuple[int, int]:
    """(height, width) from the file header, without decoding the pixels."""
    from PIL import Image
    try:
        with Image.open(io.BytesIO(data)) as img:
            return img.height, img.width
    except Exception as e:                                     # PIL raises many types
        raise VisionError(f"cannot decode image: {e}") from None


def load_image(data: bytes, spec: VisionSpec, max_pixels: Optional[int] = None) -> ImageInput:
    """Decode PNG / JPEG / WebP bytes, convert to RGB (transparent pixels over white) and
    resize to the grid geometry."""
    from PIL import Image
    try:
        img = Image.open(io.BytesIO(data))
        img.load()
    except Exception as e:                                     # PIL raises many types
        raise VisionError(f"cannot decode image: {e}") from None
    if img.mode in ("RGBA", "LA", "P"):
        rgba = img.convert("RGBA")
        base = Image.new("RGB", rgba.size, (255, 255, 255))
        base.paste(rgba, mask=rgba.split()[3])
        img = base
    else:
        img = img.convert("RGB")
    factor = spec.patch_size * spec.merge_size
    h, w = smart_resize(img.height, img.width, factor, spec.min_pixels,
                        min(max_pixels or spec.max_pixels, spec.max_pixels))
    img = img.resize((w, h), Image.BICUBIC)
    return ImageInput(h // spec.patch_size, w // spec.patch_size, np.asarray(img, dtype=np.uint8))


def pack_pixels(spec: VisionSpec, image: ImageInput) -> torch.Tensor:
    """float32 [patches, patch_values] in checkpoint order: merge blocks row-major, the
    merge x merge patches of a block, then channel, temporal copy, y, x; values rgb/127.5 - 1."""
    feature_count(spec, image)
    p, m, t = spec.patch_size, spec.merge_size, spec.temporal_patch_size
    gh, gw = image.grid_height, image.grid_width
    x = torch.from_numpy(np.array(image.rgb, copy=True)).float() / 127.5 - 1.0   # [H, W, 3]
    x = x.view(gh // m, m, p, gw // m, m, p, 3)           # br, ir, y, bc, ic, x, ch
    x = x.permute(0, 3, 1, 4, 6, 2, 5)                    # br, bc, ir, ic, ch, y, x
    x = x.reshape(gh * gw, 3, 1, p, p).expand(-1, -1, t, -1, -1)
    return x.reshape(gh * gw, spec.patch_values).contiguous()


def patch_coordinates(spec: VisionSpec, gh: int, gw: int) -> torch.Tensor:
    """int64 [patches, 2] (row, column) of each packed patch."""
    m = spec.merge_size
    br, bc, ir, ic = torch.meshgrid(torch.arange(gh // m), torch.arange(gw // m),
                                    torch.arange(m), torch.arange(m), indexing="ij")
    return torch.stack([(br * m + ir).reshape(-1), (bc * m + ic).reshape(-1)], dim=1)


# ------------------------------------------------------------------ MRoPE
def mrope_sections(half_dim: int) -> Tuple[int, int, int]:
    """(t, h, w) frequency counts; 32 frequencies split 11 / 11 / 10."""
    w = half_dim // 3
    h = (half_dim - w) // 2
    return half_dim - w - h, h, w


def mrope_positions(spec: VisionSpec, tokens: Sequence[int], spans: Sequence[Tuple[int, int]],
                    grids: Sequence[Tuple[int, int]]) -> Tuple[np.ndarray, int]:
    """int32 [3, len(tokens)] (t, h, w) rotary positions and the delta to add to a later
    token's index to get its rotary position.  Text advances all three axes together; an image
    holds t at its start position and spreads h / w over its merged grid; the text after it
    resumes at the largest position used plus one."""
    n = len(tokens)
    pos = np.zeros((3, n), dtype=np.int32)
    cursor, at = 0, 0                      # token index, next rotary position
    for (start, end), (gh, gw) in zip(spans, grids):
        run = start - cursor
        pos[:, cursor:start] = at + np.arange(run, dtype=np.int32)
        at += run
        mh, mw = gh // spec.merge_size, gw // spec.merge_size
        if mh * mw != end - start:
            raise VisionError("image span does not match its grid")
        pos[0, start:end] = at
        pos[1, start:end] = at + np.repeat(np.arange(mh, dtype=np.int32), mw)
        pos[2, start:end] = at + np.tile(np.arange(mw, dtype=np.int32), mh)
        at += max(mh, mw)
        cursor = end
    pos[:, cursor:] = at + np.arange(n - cursor, dtype=np.int32)
    return pos, (at + (n - cursor)) - n


def mrope_tables(positions: torch.Tensor, head_dim: int, theta: float):
    """cos / sin [rows, head_dim / 2] fp32 for interleaved MRoPE: frequency i reads the h axis
    when ``i % 3 == 1`` and the w axis when ``i % 3 == 2`` (inside their section counts), the
    t axis otherwise.  With equal axes this is the ordinary rotary table."""
    half = head_dim // 2
    _, sh, sw = mrope_sections(half)
    idx = torch.arange(half, device=positions.device)
    axis = torch.zeros(half, dtype=torch.long, device=positions.device)
    axis[(idx % 3 == 1) & (idx < 3 * sh)] = 1
    axis[(idx % 3 == 2) & (idx < 3 * sw)] = 2
    inv = theta ** (-torch.arange(0, head_dim, 2, dtype=torch.float64,
                                  device=positions.device) / head_dim)
    p = positions.double()[axis]                           # [half, rows]
    ang = p.t() * inv[None, :]
    return ang.cos().float(), ang.sin().float()


# ------------------------------------------------------------------ encoder
class VisionEncoder(torch.nn.Module):
    """Patch projection, 2-D rotary self-attention blocks over one image, and the 2x2 merger
    projecting to the decoder width.  Weights are random-init from a seed (no converter from a
    checkpoint tower exists yet); the layout is the one a converted tower would fill."""

    def __init__(self, spec: VisionSpec, seed: int = 0):
        super().__init__()
        self.spec = spec
        g = torch.Generator().manual_seed(seed)
        w, d = spec.width, spec.width // spec.heads
        if d % 4:
            raise VisionError("encoder head size must be a multiple of 4 for 2-D rotary")

        def lin(o, i):
            return torch.nn.Parameter(torch.randn(o, i, generator=g) * (i ** -0.5))

        self.patch = lin(w, spec.patch_values)
        self.blocks = torch.nn.ModuleList()
        for _ in range(spec.depth):
            b = torch.nn.Module()
            b.n1, b.n2 = torch.nn.LayerNorm(w), torch.nn.LayerNorm(w)
            b.qkv, b.out = lin(3 * w, w), lin(w, w)
            b.up, b.down = lin(4 * w, w), lin(w, 4 * w)
            self.blocks.append(b)
        m2 = spec.merge_size ** 2
        self.norm = torch.nn.LayerNorm(w)
        self.m1, self.m2 = lin(w * m2, w * m2), lin(spec.hidden, w * m2)
        self.requires_grad_(False)

    def _rope(self, coords: torch.Tensor, d: int):
        quarter = d // 4
        inv = 10000.0 ** (-torch.arange(quarter, dtype=torch.float32, device=coords.device)
                          / quarter)
        ang = torch.cat([coords[:, :1].float() * inv, coords[:, 1:].float() * inv], dim=1)
        return ang.cos(), ang.sin()                         # [patches, d / 2]

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        """pixels [patches, patch_values] (packed order) -> features [patches / merge^2, hidden]."""
        s = self.spec
        dt = self.patch.dtype
        x = pixels.to(dt) @ self.patch.t()
        n, heads, d = x.shape[0], s.heads, s.width // s.heads
        cos, sin = self._rope(patch_coordinates(s, gh, gw).to(x.device), d)
        cos, sin = cos.to(dt)[:, None, :], sin.to(dt)[:, None, :]

        def rot(t):
            a, b = t[..., :d // 2], t[..., d // 2:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

        for b in self.blocks:
            q, k, v = (b.n1(x) @ b.qkv.t()).view(n, 3, heads, d).unbind(1)
            att = torch.nn.functional.scaled_dot_product_attention(
                rot(q).transpose(0, 1), rot(k).transpose(0, 1), v.transpose(0, 1))
            x = x + att.transpose(0, 1).reshape(n, -1) @ b.out.t()
            x = x + torch.nn.functional.gelu(b.n2(x) @ b.up.t()) @ b.down.t()
        x = self.norm(x).view(n // s.merge_size ** 2, -1)   # merge blocks are contiguous
        return torch.nn.functional.gelu(x @ self.m1.t()) @ self.m2.t()

    def encode(self, image: ImageInput) -> torch.Tensor:
        dev = self.patch.device
        return self(pack_pixels(self.spec, image).to(dev), image.grid_height, image.grid_width)


class FeatureCache:
    """Encoder outputs keyed by image digest (not by token position), least recently used
    entries dropped above a byte budget."""

    def __init__(self, budget_bytes: int = 256 << 20):
        self.budget = budget_bytes
        self.bytes = 0
        self.hits = self.misses = 0
        self._items: "OrderedDict[int, torch.Tensor]" = OrderedDict()

    def get(self, image: ImageInput, encoder: VisionEncoder) -> torch.Tensor:
        key = image.digest()
        hit = self._items.get(key)
        if hit is not None:
            self._items.move_to_end(key)
            self.hits += 1
            return hit
        self.misses += 1
        feats = encoder.encode(image)
        size = feats.numel() * feats.element_size()
        if size <= self.budget:
            self._items[key] = feats
            self.bytes += size
            while self.bytes > self.budget:
                _, old = self._items.popitem(last=False)
                self.bytes -= old.numel() * old.element_size()
        return feats
