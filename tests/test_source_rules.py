"""Repository rules that a kernel or a comment can break silently: no cluster-multicast bulk loads anywhere,
none of the batched-memcpy driver calls, no disassembler or clock-setting invocations, nothing that kills
processes by pattern, and comments that stand on their own (no build-note file names, no machine paths)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXT = (".py", ".cu", ".cuh", ".h", ".sh", ".yaml", ".toml")


def _files():
    for top in ("axon_b200", "axon", "csrc", "tests", "bench.py", "__graft_entry__.py", "baseline"):
        p = os.path.join(ROOT, top)
        if os.path.isfile(p):
            yield p
        for d, dirs, names in os.walk(p):
            dirs[:] = [x for x in dirs if x not in ("__pycache__", "_ref", "build")]
            for n in names:
                if n.endswith(EXT):
                    yield os.path.join(d, n)


def _j(*parts):          # the patterns are assembled so that this file does not contain them itself
    return "".join(parts)


FORBIDDEN = {
    "bulk load with cluster multicast": re.compile(_j(r"\.multi", r"cast::clu", "ster")),
    "batched memcpy driver call": re.compile(_j("Memcpy", "(3D)?", "Batch", "Async")),
    "disassembler": re.compile(_j(r"\b(cuobj", "dump|nvdis", "asm|objdump", r"\s+-d)\b")),
    "clock / power setting": re.compile(_j(r"nvidia-smi\s+(-", "lgc|-", "ac|-", "pm|-", "pl|--lock)")),
    "kill by pattern": re.compile(_j(r"\b(pk", "ill|kill", "all)", r"\b")),
    "device trap": re.compile(_j(r"__tr", r"ap\s*\(")),
    "build-note reference": re.compile(_j(r"\b(SUR", "VEY|VER", "DICT|ADV", r"ICE|DES", r"IGN|BASE", r"LINE)\.md\b")),
    "machine path": re.compile(_j(r"/ro", r"ot/(re", "po|refe", "rence)")),
    "job runner name": re.compile(_j(r"\bgpu", r"run\b")),
}


def test_sources_follow_the_repository_rules():
    bad = []
    for path in _files():
        rel = os.path.relpath(path, ROOT)
        with open(path, encoding="utf-8", errors="replace") as f:
            for i, line in enumerate(f, 1):
                for what, rx in FORBIDDEN.items():
                    if rx.search(line):
                        bad.append(f"{rel}:{i}: {what}: {line.strip()[:100]}")
    assert not bad, "\n".join(bad[:40])
