"""FrozenLake as a multi-turn text environment (task of the reference's quick-start recipe:
recipes/frozenlake/env.py, which wraps Gymnasium's toy-text FrozenLake).

The grid world is implemented here directly (no Gymnasium dependency): ``S`` start, ``F`` frozen, ``H`` hole,
``G`` goal; actions 1 = left, 2 = down, 3 = right, 4 = up; with ``is_slippery`` the move goes in the intended
direction with probability ``p`` and sideways otherwise. A map comes from a seed: cells are frozen with
probability ``p_frozen`` and the map is redrawn until the goal is reachable from the start within ``max_steps``
moves. Reward 1 on reaching the goal; the episode ends on goal, hole or after ``max_steps`` actions.

Observations are the rendered grid as text: ``P`` player, ``_`` frozen, ``O`` hole, ``G`` goal, ``X`` player in a
hole, ``√`` player on the goal."""
from __future__ import annotations

import numpy as np

from axon_b200.core.env import BaseEnv, register_env

MAX_STEPS = 5
MOVES = {1: (0, -1), 2: (1, 0), 3: (0, 1), 4: (-1, 0)}          # left, down, right, up as (row, col) deltas
SYMBOLS = {"P": " P ", "F": " _ ", "H": " O ", "G": " G ", "X": " X ", "W": " √ "}


def reachable(board: list[list[str]], limit: int) -> bool:
    """Breadth-first search: is ``G`` within ``limit`` moves of ``S`` without stepping on a hole?"""
    n = len(board)
    start = next((r, c) for r in range(n) for c in range(n) if board[r][c] == "S")
    seen, frontier = {start}, [start]
    for _ in range(limit):
        nxt = []
        for r, c in frontier:
            for dr, dc in MOVES.values():
                rr, cc = r + dr, c + dc
                if not (0 <= rr < n and 0 <= cc < n) or (rr, cc) in seen or board[rr][cc] == "H":
                    continue
                if board[rr][cc] == "G":
                    return True
                seen.add((rr, cc))
                nxt.append((rr, cc))
        frontier = nxt
    return False


def generate_random_map(size: int = 8, p: float = 0.8, seed: int = 0, max_steps: int = MAX_STEPS) -> list[str]:
    """A ``size x size`` map with a goal reachable within ``max_steps`` moves, determined by ``seed``."""
    rng = np.random.default_rng(seed)
    p = min(1.0, p)
    while True:
        board = rng.choice(["F", "H"], (size, size), p=[p, 1 - p]).tolist()
        cells = rng.choice(size * size, 2, replace=False)
        (sr, sc), (gr, gc) = divmod(int(cells[0]), size), divmod(int(cells[1]), size)
        board[sr][sc], board[gr][gc] = "S", "G"
        if reachable(board, max_steps):
            return ["".join(row) for row in board]


@register_env("frozenlake")
class FrozenLakeEnv(BaseEnv):
    def __init__(self, size: int = 8, p: float = 0.8, seed: int = 42, is_slippery: bool = False, slip_p: float = 1.0 / 3.0,
                 max_steps: int = MAX_STEPS, desc: list[str] | None = None, **_):
        self.size, self.p, self.seed, self.is_slippery, self.slip_p, self.max_steps = size, p, seed, is_slippery, slip_p, max_steps
        self.desc = [list(r) for r in (desc or generate_random_map(size, p, seed, max_steps))]
        self.rng = np.random.default_rng(seed + 1)
        self.pos = self._find("S")
        self.steps = 0

    def _find(self, ch: str) -> tuple[int, int]:
        return next((r, c) for r, row in enumerate(self.desc) for c, x in enumerate(row) if x == ch)

    def reset(self):
        self.pos, self.steps = self._find("S"), 0
        self.rng = np.random.default_rng(self.seed + 1)
        return self.render(), {}

    def cell(self) -> str:
        return self.desc[self.pos[0]][self.pos[1]]

    def finished(self) -> bool:
        return self.cell() in "GH"

    def success(self) -> bool:
        return self.cell() == "G"

    def step(self, action):
        """``action``: 1..4 (anything else, including an unparsable response, is an invalid move that costs a turn)."""
        self.steps += 1
        out_of_turns = self.steps >= self.max_steps
        if self.finished():
            return self.render(), float(self.success()), True, {"action_is_effective": False}
        if action not in MOVES:
            return self.render(), 0.0, out_of_turns, {"action_is_effective": False}
        a = int(action)
        if self.is_slippery and self.rng.random() > 1.0 - 2 * self.slip_p:
            a = {1: (2, 4), 2: (1, 3), 3: (2, 4), 4: (1, 3)}[a][int(self.rng.integers(2))]      # slide sideways
        dr, dc = MOVES[a]
        r, c = min(max(self.pos[0] + dr, 0), len(self.desc) - 1), min(max(self.pos[1] + dc, 0), len(self.desc) - 1)
        moved = (r, c) != self.pos
        self.pos = (r, c)
        done = self.finished() or out_of_turns
        return self.render(), float(self.success()), done, {"action_is_effective": moved}

    def render(self) -> str:
        rows = []
        for r, row in enumerate(self.desc):
            cells = []
            for c, x in enumerate(row):
                x = "F" if x == "S" else x
                if (r, c) == self.pos:
                    x = {"H": "X", "G": "W"}.get(x, "P")
                cells.append(SYMBOLS[x])
            rows.append("".join(cells))
        return "\n".join(rows)

    @staticmethod
    def from_dict(env_info: dict) -> "FrozenLakeEnv":
        keys = ("size", "p", "seed", "is_slippery", "slip_p", "max_steps", "desc")
        return FrozenLakeEnv(**{k: env_info[k] for k in keys if k in env_info})
