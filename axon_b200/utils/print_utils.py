"""Console helpers (reference: axon/utils/print_utils.py:26-95)."""
from __future__ import annotations

import click


def colorful_print(string: str, *args, **kwargs) -> None:
    fg = args[0] if args else kwargs.pop("fg", None)
    click.secho(string, fg=fg, **{k: v for k, v in kwargs.items() if k in ("bold", "bg", "underline")})


def colorful_warning(string: str, *args, **kwargs) -> None:
    colorful_print(f"[warning] {string}", *(args or ("yellow",)), **kwargs)


def log_metrics(metrics: dict, title: str = "Metrics", color: str = "white") -> None:
    colorful_print(f"== {title}", color, bold=True)
    for k in sorted(metrics):
        v = metrics[k]
        colorful_print(f"  {k}: {v:.6g}" if isinstance(v, float) else f"  {k}: {v}", color)


def merge_dicts(dict_list: list[dict]) -> dict[str, list]:
    out: dict[str, list] = {}
    for d in dict_list:
        for k, v in d.items():
            out.setdefault(k, []).append(v)
    return out


def append_to_dict(data: dict, new_data: dict, prefix: str = "") -> None:
    for k, v in new_data.items():
        data.setdefault(prefix + k, []).append(v)
