"""Image / video inputs of multimodal prompts (reference: axon/utils/vision_utils.py:22-130).

``process_image`` accepts a PIL image or a dict (``{"image": PIL | path | file:// url | data: url}`` or
``{"bytes": ...}``, optional ``min_pixels`` / ``max_pixels`` / ``resized_height`` / ``resized_width``)
and returns an RGB image whose sides are multiples of ``2 * image_patch_size`` (one merged 2x2 patch of
the Qwen-VL family) with the pixel count inside the bounds, aspect ratio kept as closely as the grid
allows. ``process_video`` does the same for a list of frames (decoding of video containers needs a codec
library that is not part of this package: pass frames)."""
from __future__ import annotations

import base64
import math
from io import BytesIO

from PIL import Image

MIN_PIXELS = 4 * 28 * 28
MAX_PIXELS = 16384 * 28 * 28
MAX_RATIO = 200


def get_image(image_path: str) -> Image.Image:
    with Image.open(image_path) as img:
        return img.convert("RGB")


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = MIN_PIXELS, max_pixels: int = MAX_PIXELS) -> tuple[int, int]:
    """Sides rounded to multiples of ``factor`` with ``min_pixels <= h * w <= max_pixels``."""
    if max(height, width) / max(1, min(height, width)) > MAX_RATIO:
        raise ValueError(f"aspect ratio must be below {MAX_RATIO}, got {max(height, width) / min(height, width):.1f}")
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


def _open(src) -> Image.Image:
    if isinstance(src, Image.Image):
        return src
    if isinstance(src, (bytes, bytearray)):
        return Image.open(BytesIO(src))
    if isinstance(src, str):
        if src.startswith("data:image") and "base64," in src:
            return Image.open(BytesIO(base64.b64decode(src.split("base64,", 1)[1])))
        if src.startswith("file://"):
            src = src[len("file://"):]
        if src.startswith(("http://", "https://")):
            raise ValueError("remote images are not fetched here; pass bytes or a local path")
        return Image.open(src)
    raise TypeError(f"cannot read an image from {type(src).__name__}")


def process_image(image, image_patch_size: int = 14) -> Image.Image:
    if isinstance(image, Image.Image):
        return image.convert("RGB")
    image = dict(image)
    if "bytes" in image:
        assert "image" not in image, "Cannot have both `bytes` and `image`"
        image["image"] = Image.open(BytesIO(image["bytes"]))
    img = _open(image.get("image", image.get("image_url"))).convert("RGB")
    factor = 2 * image_patch_size
    if "resized_height" in image and "resized_width" in image:
        h, w = smart_resize(int(image["resized_height"]), int(image["resized_width"]), factor)
    else:
        h, w = smart_resize(img.height, img.width, factor, int(image.get("min_pixels", MIN_PIXELS)), int(image.get("max_pixels", MAX_PIXELS)))
    return img if (img.height, img.width) == (h, w) else img.resize((w, h), Image.BICUBIC)


def process_video(video: dict, image_patch_size: int = 14, nframes: int | None = None, fps: float | None = None,
                  fps_min_frames: int | None = None, fps_max_frames: int | None = None):
    """Frames of ``video["video"]`` (a list of images / paths) sampled to ``nframes`` (or every frame),
    rounded down to an even count, each through ``process_image`` with one shared target size."""
    frames = video.get("video")
    if not isinstance(frames, (list, tuple)):
        raise ValueError("pass the video as a list of frames: {'type': 'video', 'video': [frame, ...]}")
    n = len(frames)
    want = nframes or n
    if fps_min_frames:
        want = max(want, fps_min_frames)
    if fps_max_frames:
        want = min(want, fps_max_frames)
    want = max(2, min(n, want) // 2 * 2) if n >= 2 else n
    idx = [round(i * (n - 1) / max(1, want - 1)) for i in range(want)]
    first = _open(frames[idx[0]])
    h, w = smart_resize(first.height, first.width, 2 * image_patch_size, int(video.get("min_pixels", MIN_PIXELS)), int(video.get("max_pixels", MAX_PIXELS)))
    return [process_image({"image": frames[i], "resized_height": h, "resized_width": w}, image_patch_size) for i in idx]
