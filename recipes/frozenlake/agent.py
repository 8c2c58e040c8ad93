"""Agent for the FrozenLake recipe (reference: recipes/frozenlake/agent.py): explains the grid symbols and the
answer format in the system prompt, shows the current grid every turn, and reads the move out of the last fenced
block (``` ... ```) of the model's response: a direction word or its number."""
from __future__ import annotations

import re

from axon_b200.core.agent import Action, BaseAgent, register_agent, split_thought

DIRECTIONS = {"left": 1, "down": 2, "right": 3, "up": 4}

SYSTEM_PROMPT = """You are walking on a frozen lake and must reach the goal without falling into a hole.

Symbols: _ frozen surface (safe), O hole (the episode ends), G goal, P your position. X means you fell into a hole, √ means you reached the goal.
Rows are listed top to bottom, columns left to right. Moving against the border leaves you where you are.

Each turn, reason briefly about the positions of P, G and the holes, then give exactly one move, Left, Down, Right or Up, between triple backticks, for example ```Right```. Avoid moves that do not change your position, and do not repeat a plan that already failed."""


@register_agent("frozenlake")
class FrozenLakeAgent(BaseAgent):
    def __init__(self, max_turns: int = 5, show_history: bool = True):
        self.max_turns, self.show_history = max_turns, show_history
        self.reset()

    @property
    def system_prompt(self) -> str:
        return SYSTEM_PROMPT

    def reset(self) -> None:
        self.turn = 0
        self.last_grid: str | None = None

    def process_observation(self, observation, reward: float, done: bool, info: dict, **kwargs) -> str:
        self.turn += 1
        grid = str(observation)
        note = ""
        if self.last_grid is not None and grid == self.last_grid and not done:
            note = "Your last move had no effect (invalid answer, or a move against the border). Choose a different move.\n"
        self.last_grid = grid
        left = max(0, self.max_turns - self.turn + 1)
        return f"{note}Current grid (turn {self.turn}, {left} moves left):\n{grid}\nGive your next move between triple backticks."

    def process_action(self, action: str) -> Action:
        thought, rest = split_thought(action)
        blocks = re.findall(r"```(.*?)```", rest, flags=re.DOTALL)
        move = 0
        if blocks:
            text = blocks[-1].strip().lower()
            if text in DIRECTIONS:
                move = DIRECTIONS[text]
            elif text.isdigit() and int(text) in DIRECTIONS.values():
                move = int(text)
            else:
                words = [w for w in re.findall(r"[a-z]+", text) if w in DIRECTIONS]
                move = DIRECTIONS[words[-1]] if words else 0
        return Action(thought=thought or rest, action=move)
