from .base_program import PROGRAM_CLASS_MAPPING, BaseProgram, ProgramResult, register_program
from .proxy_program import ProxyProgram
from .react_program import ReactProgram
from .external import NemoGymProgram, VerifiersProgram  # noqa: F401  (registers "nemo_gym" and "verifiers")

__all__ = ["BaseProgram", "ProgramResult", "ReactProgram", "ProxyProgram", "PROGRAM_CLASS_MAPPING", "register_program"]
