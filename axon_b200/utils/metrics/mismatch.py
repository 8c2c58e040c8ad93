"""How far the trainer's log-probs of the sampled tokens are from the sampler's own
(reference: axon/utils/metrics/trainer_sampler_mismatch_metrics.py:36-146). Returned as sufficient
statistics so shards from several workers aggregate exactly."""
from __future__ import annotations

import torch

_READABLE = ("batch/sampler_probs_diff_max", "batch/sampler_probs_diff_mean", "batch/sampler_probs_diff_min",
             "batch/sampler_probs_diff_std", "batch/sampler_logprobs_diff_max", "batch/sampler_logprobs_diff_mean",
             "batch/sampler_logprobs_diff_min", "batch/sampler_logprobs_diff_std", "batch/sampler_actor_probs_pearson_corr")


def compute_trainer_sampler_mismatch_metrics(batch) -> dict:
    mask = batch.batch["response_mask"].bool()
    a_lp, s_lp = batch.batch["old_log_probs"].float(), batch.batch["sampler_log_probs"].float()
    if not mask.any():
        return {"batch/sampler_probs_diff_max": 0.0, "batch/sampler_probs_diff_min": 0.0, "batch/sampler_logprobs_diff_max": 0.0,
                "batch/sampler_logprobs_diff_min": 0.0, "_valid_count": 0}
    a, s = a_lp.exp()[mask].double(), s_lp.exp()[mask].double()
    dp, dl = (a - s).abs(), (a_lp - s_lp).abs()[mask].double()
    f = lambda t: float(t.item())                                    # noqa: E731
    return {"batch/sampler_probs_diff_max": f(dp.max()), "batch/sampler_probs_diff_min": f(dp.min()),
            "batch/sampler_logprobs_diff_max": f(dl.max()), "batch/sampler_logprobs_diff_min": f(dl.min()),
            "_valid_count": int(mask.sum()), "_sum": f(dp.sum()), "_sum_squares": f((dp ** 2).sum()),
            "_logprobs_sum": f(dl.sum()), "_logprobs_sum_squares": f((dl ** 2).sum()), "_actor_sum": f(a.sum()),
            "_sampler_sum": f(s.sum()), "_actor_sum_squares": f((a ** 2).sum()), "_sampler_sum_squares": f((s ** 2).sum()),
            "_product_sum": f((a * s).sum())}


def aggregate_trainer_sampler_metrics(metrics_list: list[dict]) -> dict:
    if not metrics_list:
        return {}
    tot = lambda k: sum(m.get(k, 0.0) for m in metrics_list)          # noqa: E731
    n = tot("_valid_count")
    if n == 0:
        return {k: 0.0 for k in _READABLE}
    mean, lmean = tot("_sum") / n, tot("_logprobs_sum") / n
    var, lvar = tot("_sum_squares") / n - mean ** 2, tot("_logprobs_sum_squares") / n - lmean ** 2
    am, sm = tot("_actor_sum") / n, tot("_sampler_sum") / n
    a_sd = max(0.0, tot("_actor_sum_squares") / n - am ** 2) ** 0.5
    s_sd = max(0.0, tot("_sampler_sum_squares") / n - sm ** 2) ** 0.5
    cov = tot("_product_sum") / n - am * sm
    live = [m for m in metrics_list if m.get("_valid_count", 0) > 0]
    return {"batch/sampler_probs_diff_max": max(m["batch/sampler_probs_diff_max"] for m in live),
            "batch/sampler_probs_diff_mean": mean,
            "batch/sampler_probs_diff_min": min(m["batch/sampler_probs_diff_min"] for m in live),
            "batch/sampler_probs_diff_std": var ** 0.5 if var > 0 else 0.0,
            "batch/sampler_logprobs_diff_max": max(m["batch/sampler_logprobs_diff_max"] for m in live),
            "batch/sampler_logprobs_diff_mean": lmean,
            "batch/sampler_logprobs_diff_min": min(m["batch/sampler_logprobs_diff_min"] for m in live),
            "batch/sampler_logprobs_diff_std": lvar ** 0.5 if lvar > 0 else 0.0,
            "batch/sampler_actor_probs_pearson_corr": cov / (a_sd * s_sd) if a_sd * s_sd > 0 else 0.0}
