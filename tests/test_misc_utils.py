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


def test_precision_names_device_helpers_and_padding_round_trip(capsys):
    import logging

    import torch

    from axon_b200 import globals as G
    from axon_b200.trainer.algos.constants import VALID_BATCH_REDUCE, VALID_TOKEN_REDUCE
    from axon_b200.utils.logger import DecoratorLoggerBase, LocalLogger, concat_dict_to_str, print_with_rank
    from axon_b200.utils.torch.attention import pad_input, unpad_input
    from axon_b200.utils.torch.device import get_device_name, get_nccl_backend, get_torch_device
    from axon_b200.utils.torch.dtypes import PrecisionType
    assert PrecisionType.to_dtype("bf16") is torch.bfloat16 and PrecisionType.to_dtype(16) is torch.float16
    assert PrecisionType.to_dtype(torch.float32) is torch.float32 and PrecisionType.to_str(torch.bfloat16) == "bf16"
    assert PrecisionType.is_bf16("bfloat16") and not PrecisionType.is_fp16("bf16") and PrecisionType.supported_type("mixed")
    assert get_device_name() in ("cuda", "cpu") and get_nccl_backend() in ("nccl", "gloo") and hasattr(get_torch_device(), "synchronize")
    assert "token-mean" in VALID_BATCH_REDUCE and "mean-norm" in VALID_TOKEN_REDUCE and G.THOUGHT_DELIMITER_END == "</think>"
    x = torch.arange(2 * 5 * 3, dtype=torch.float32).view(2, 5, 3)
    mask = torch.tensor([[1, 1, 1, 0, 0], [1, 1, 1, 1, 1]])
    packed, idx, cu, longest, lens = unpad_input(x, mask)
    assert packed.shape == (8, 3) and cu.tolist() == [0, 3, 8] and longest == 5 and lens.tolist() == [3, 5]
    back = pad_input(packed, idx, 2, 5)
    assert torch.equal(back, x * mask[..., None])
    assert concat_dict_to_str({"a": 1, "b": "text", "c": 0.5}, 3) == "step:3 - a:1 - c:0.5"
    LocalLogger().log({"loss": 1.5}, step=2)
    DecoratorLoggerBase("actor", rank=1).logging_function("hidden")          # rank 1 stays quiet
    DecoratorLoggerBase("actor", rank=0).logging_function("shown")
    print_with_rank("hello", rank=3)
    out = capsys.readouterr().out
    assert "step:2 - loss:1.5" in out and "actor shown" in out and "hidden" not in out and "[Rank 3] hello" in out
    DecoratorLoggerBase("x", logger=logging.getLogger("t"), level=logging.INFO).logging_function("via logging")


def test_math_grading_normalises_and_compares_symbolically():
    from axon_b200.utils.rewards import RewardConfig, math_reward_fn
    from axon_b200.utils.rewards.math_grading import extract_answer, grade_answer as g
    same = [("\\frac12", "1/2"), ("0.5", "\\frac{1}{2}"), ("\\dfrac{3}{4}", "0.75"), ("5 cm", "5"), ("30^\\circ", "30"), ("x = 5", "5"),
            ("1,234", "1234"), ("\\$12.50", "12.5"), ("2\\sqrt{3}", "\\sqrt{12}"), ("(1, 2)", "(1,2)"), ("\\{1,2,3\\}", "\\{3,2,1\\}"),
            ("3, 1", "1, 3"), ("x^2+2x+1", "(x+1)^2"), ("\\frac{\\pi}{2}", "pi/2"), ("\\text{seven}", "7"), ("10\\%", "10"),
            ("2^{10}", "1024"), ("\\sqrt2", "\\sqrt{2}"), ("12 square units", "12"), ("3.0", "3"), ("[0,1)", "[0,1)"), ("\\infty", "oo"),
            ("\\frac{1}{3}", "0.3333333333")]
    different = [("(1,2)", "[1,2]"), ("7", "8"), ("\\frac{1}{3}", "0.33"), ("abc", "abd"), ("(1,2)", "(2,1)"), ("x+1", "x+2"), ("", "1")]
    assert [p for p in same if not g(*p)] == []
    assert [p for p in different if g(*p)] == []
    assert extract_answer("so the final answer is 42.") == "42" and extract_answer("x \\boxed{\\frac{1}{2}} y") == "\\frac{1}{2}"
    cfg = RewardConfig()
    ok = math_reward_fn({"ground_truth": ["\\frac{\\sqrt{12}}{2}"]}, "<think>hm</think> thus \\boxed{\\sqrt{3}}", cfg)
    assert ok.is_correct and ok.reward == cfg.correct_reward
    assert not math_reward_fn({"ground_truth": "4"}, "\\boxed{5}", cfg).is_correct
    assert math_reward_fn({"ground_truth": "4"}, "no answer here", cfg).reward == cfg.format_error_reward
