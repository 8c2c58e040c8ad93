"""Child-process clean-up (reference: axon/utils/process.py)."""
from __future__ import annotations


def cleanup_subprocesses(process_list: list) -> None:
    """Join finished children; terminate (then kill) the ones still alive. Only handles passed in."""
    for p in process_list:
        if p.is_alive():
            p.terminate()
    for p in process_list:
        p.join(timeout=5)
        if p.is_alive():
            p.kill()
            p.join(timeout=5)
    process_list.clear()
