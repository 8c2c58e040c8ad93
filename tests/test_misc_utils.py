"""Retrieval helper and image preprocessing."""
import io

import pytest
from PIL import Image

from axon_b200.utils.rag_utils import RAG, HashedNgramEncoder
from axon_b200.utils.vision_utils import process_image, process_video, smart_resize


def test_rag_retrieves_lexically_closest_document():
    docs = ["The integral of x squared is x cubed over three.", "Paris is the capital of France.", "Binary search runs in logarithmic time."]
    rag = RAG(docs, encoder=HashedNgramEncoder())
    top = rag.top_k("what is the capital city of France?", k=2)
    assert top[0]["idx"] == 1 and top[0]["text"] == docs[1] and float(top[0]["score"]) > float(top[1]["score"])
    assert rag.top_k("logarithmic binary search", k=1)[0]["idx"] == 2


def test_smart_resize_bounds_and_grid():
    h, w = smart_resize(1000, 700, 28, 4 * 28 * 28, 256 * 28 * 28)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 256 * 28 * 28 and abs(h / w - 1000 / 700) < 0.1
    h, w = smart_resize(10, 10, 28, 4 * 28 * 28, 256 * 28 * 28)
    assert h * w >= 4 * 28 * 28
    with pytest.raises(ValueError):
        smart_resize(10, 10000)


def test_process_image_and_video():
    img = Image.new("L", (333, 217), 128)
    buf = io.BytesIO(); img.save(buf, format="PNG")
    out = process_image({"bytes": buf.getvalue(), "max_pixels": 64 * 28 * 28})
    assert out.mode == "RGB" and out.width % 28 == 0 and out.height % 28 == 0 and out.width * out.height <= 64 * 28 * 28
    frames = [Image.new("RGB", (120, 90), (i * 20, 0, 0)) for i in range(7)]
    vid = process_video({"type": "video", "video": frames}, nframes=4)
    assert len(vid) == 4 and len({f.size for f in vid}) == 1 and vid[0].size[0] % 28 == 0
