"""Bounded image input and deterministic Qwen2-VL-compatible patching (CPU image maths, no graphics API).

Accepts PNG / JPEG / WebP / GIF (single frame) up to 32 MiB encoded, from bytes, a canonical base64 data URL or
a local path; the declared MIME type must agree with the magic bytes.  The RGB raster (EXIF orientation ignored)
is resized with a Catmull-Rom (bicubic) filter to multiples of patch x merge = 32 pixels inside
[65,536, 16,777,216] pixels, normalised to (v / 255 - 0.5) / 0.5 and cut into patches of 3 x 2 x 16 x 16 values
ordered by 2x2 merge block, so that every four consecutive rows form one visual token.  At most 2 images and
16,384 visual tokens per request (reference: crates/sllm-frontend/src/vision.rs:13-20 limits, :219-300 patch
order, :366-385 smart resize).
"""
from __future__ import annotations

import base64
import hashlib
import io
import math
import os
from dataclasses import dataclass

import numpy as np

MAX_ENCODED_IMAGE_BYTES = 32 * 1024 * 1024
MIN_IMAGE_PIXELS = 65_536
MAX_IMAGE_PIXELS = 16_777_216
PATCH, TEMPORAL, MERGE = 16, 2, 2
MAX_IMAGE_COUNT = 2
MAX_TOTAL_VISUAL_TOKENS = 16_384
MAX_ASPECT = 200.0
_MAGIC = {"image/png": (b"\x89PNG\r\n\x1a\n",), "image/jpeg": (b"\xff\xd8\xff",), "image/gif": (b"GIF87a", b"GIF89a"),
          "image/webp": (b"RIFF",)}


class VisionError(ValueError):
    pass


def _sniff(data: bytes) -> str:
    for mime, magics in _MAGIC.items():
        if any(data.startswith(m) for m in magics) and (mime != "image/webp" or data[8:12] == b"WEBP"):
            return mime
    raise VisionError("image format is unsupported")


@dataclass
class BoundedImage:
    data: bytes
    mime: str
    sha256: str

    @staticmethod
    def from_bytes(data: bytes) -> "BoundedImage":
        if not data or len(data) > MAX_ENCODED_IMAGE_BYTES:
            raise VisionError("encoded image exceeds the bounded size")
        return BoundedImage(bytes(data), _sniff(data), hashlib.sha256(data).hexdigest())

    @staticmethod
    def from_data_url(url: str) -> "BoundedImage":
        if not url.startswith("data:") or ";base64," not in url:
            raise VisionError("image URL is not a canonical base64 data URL")
        head, b64 = url[5:].split(";base64,", 1)
        if head not in _MAGIC or len(b64) > MAX_ENCODED_IMAGE_BYTES * 4 // 3 + 4:
            raise VisionError("image URL is not a canonical base64 data URL")
        try:
            data = base64.b64decode(b64, validate=True)
        except Exception:
            raise VisionError("image URL is not a canonical base64 data URL") from None
        if base64.b64encode(data).decode() != b64:
            raise VisionError("image URL is not a canonical base64 data URL")
        img = BoundedImage.from_bytes(data)
        if img.mime != head:
            raise VisionError("image MIME type differs from magic bytes")
        return img

    @staticmethod
    def from_local_path(path: str) -> "BoundedImage":
        try:
            if os.path.getsize(path) > MAX_ENCODED_IMAGE_BYTES:
                raise VisionError("encoded image exceeds the bounded size")
            with open(path, "rb") as f:
                return BoundedImage.from_bytes(f.read(MAX_ENCODED_IMAGE_BYTES + 1))
        except OSError:
            raise VisionError("image bytes could not be read") from None

    def decode_rgb(self) -> np.ndarray:
        """uint8 [H, W, 3]."""
        from PIL import Image
        Image.MAX_IMAGE_PIXELS = MAX_IMAGE_PIXELS * 4
        try:
            im = Image.open(io.BytesIO(self.data))
            if getattr(im, "n_frames", 1) > 1:
                raise VisionError("animated images are not accepted")
            w, h = im.size
            validate_dimensions(w, h)
            arr = np.asarray(im.convert("RGB"), dtype=np.uint8)
        except VisionError:
            raise
        except Exception:
            raise VisionError("image is malformed") from None
        return arr


def validate_dimensions(width: int, height: int) -> None:
    if width <= 0 or height <= 0 or width * height > MAX_IMAGE_PIXELS * 4:
        raise VisionError("image pixel area is out of range")
    if max(width, height) / min(width, height) > MAX_ASPECT:
        raise VisionError("image aspect ratio is out of range")


def _round_half_even(x: float) -> float:
    return float(np.round(x))          # numpy rounds half to even


def smart_resize(height: int, width: int):
    validate_dimensions(width, height)
    f = float(PATCH * MERGE)
    rh, rw = _round_half_even(height / f) * f, _round_half_even(width / f) * f
    if rh * rw > MAX_IMAGE_PIXELS:
        beta = math.sqrt(height * width / MAX_IMAGE_PIXELS)
        rh, rw = max(math.floor(height / beta / f) * f, f), max(math.floor(width / beta / f) * f, f)
    elif rh * rw < MIN_IMAGE_PIXELS:
        beta = math.sqrt(MIN_IMAGE_PIXELS / (height * width))
        rh, rw = math.ceil(height * beta / f) * f, math.ceil(width * beta / f) * f
    return int(rh), int(rw)


@dataclass
class ProcessedImage:
    resized_height: int
    resized_width: int
    grid_thw: tuple
    patches: np.ndarray          # float32 [grid_h * grid_w, 3 * 2 * 16 * 16]
    merged_positions: list       # (temporal, row, column) of every visual token
    visual_tokens: int
    patch_sha256: str
    source_sha256: str


def process_image(img: BoundedImage) -> ProcessedImage:
    from PIL import Image
    rgb = img.decode_rgb()
    h, w = rgb.shape[:2]
    rh, rw = smart_resize(h, w)
    resized = np.asarray(Image.fromarray(rgb).resize((rw, rh), Image.BICUBIC), dtype=np.uint8)
    gh, gw = rh // PATCH, rw // PATCH
    if gh % MERGE or gw % MERGE:
        raise VisionError("patch geometry is invalid")
    x = (resized.astype(np.float32) / np.float32(255.0) - np.float32(0.5)) / np.float32(0.5)      # [rh, rw, 3]
    # [block_row, merge_row, patch_row, block_col, merge_col, patch_col, channel]
    x = x.reshape(gh // MERGE, MERGE, PATCH, gw // MERGE, MERGE, PATCH, 3)
    # -> [block_row, block_col, merge_row, merge_col, channel, patch_row, patch_col]
    x = x.transpose(0, 3, 1, 4, 6, 2, 5)
    x = np.repeat(x[:, :, :, :, :, None], TEMPORAL, axis=5)          # temporal copies between channel and patch rows
    patches = np.ascontiguousarray(x).reshape(gh * gw, 3 * TEMPORAL * PATCH * PATCH)
    tokens = gh * gw // (MERGE * MERGE)
    if tokens == 0 or tokens > MAX_TOTAL_VISUAL_TOKENS:
        raise VisionError("visual token limit exceeded")
    pos = [(0, r, c) for r in range(gh // MERGE) for c in range(gw // MERGE)]
    return ProcessedImage(rh, rw, (1, gh, gw), patches, pos, tokens,
                          hashlib.sha256(patches.astype("<f4").tobytes()).hexdigest(), img.sha256)


def process_many(images: list) -> list:
    if len(images) > MAX_IMAGE_COUNT:
        raise VisionError("too many images in one request")
    out = [process_image(i) for i in images]
    if sum(p.visual_tokens for p in out) > MAX_TOTAL_VISUAL_TOKENS:
        raise VisionError("visual token limit exceeded")
    return out


def mrope_positions(text_before: int, grid_thw: tuple, text_after: int):
    """3-axis (temporal, height, width) position ids for text + one image + text, as int32 [3, T]: text tokens
    advance all three axes together; image tokens share the temporal index and enumerate the merged grid; text
    after the image continues from the largest index used so far + 1."""
    t, gh, gw = grid_thw
    mh, mw = gh // MERGE, gw // MERGE
    pos = [np.tile(np.arange(text_before, dtype=np.int32), (3, 1))]
    base = text_before
    tt = np.full(mh * mw, base, dtype=np.int32)
    hh = base + np.repeat(np.arange(mh, dtype=np.int32), mw)
    ww = base + np.tile(np.arange(mw, dtype=np.int32), mh)
    pos.append(np.stack([tt, hh, ww]))
    nxt = base + max(mh, mw)
    pos.append(np.tile(np.arange(nxt, nxt + text_after, dtype=np.int32), (3, 1)))
    return np.concatenate(pos, axis=1)
