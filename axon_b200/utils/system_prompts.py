"""System prompts used by judge rewards and the coding environments. The constant names follow the
reference (axon/utils/system_prompts.py); the wording is this project's own."""

ORM_PROMPT = """You compare two answers to a mathematics problem and decide whether they are equivalent.
Treat answers as equivalent when they denote the same mathematical object: ignore formatting, units
written differently, equivalent fractions / decimals / radicals, ordering of a set, and surrounding text.
Reply with exactly one line: [[YES]] if equivalent, [[NO]] otherwise."""

FILTER_PROOF_PROMPT = """Classify the problem given by the user into one of three categories and reply with the
category name only: PROOF (asks to prove or show something, no single final answer), MULTIPLE_CHOICE
(offers lettered or numbered options), or ANSWER (has one final answer that can be checked)."""

EXTRACT_SOLUTION_PROMPT = """Extract the final answer from the solution text as a LaTeX string. Output only the
answer: no words, no explanation, no surrounding dollar signs. If several candidate answers appear, take the
last one the solution commits to. If there is no answer, output NONE."""

REFINE_AMC_PROMPT = """Rewrite the LaTeX of the given problem so that every formula parses with a standard LaTeX
parser: balance braces, replace non-standard macros by standard ones, keep the mathematical content and the
wording unchanged. Output the corrected problem only."""

FETCH_MC_PROMPT = """You are given a multiple-choice problem and a solution. Output the letter of the option the
solution selects, and nothing else."""

LCB_SYSTEM_MESSAGE_GENERIC = ("You are an expert Python programmer. You will be given a problem specification and must write a "
                              "correct Python program that satisfies it and passes all tests.")
LCB_FORMATTING_MESSAGE_WITH_STARTER_CODE = ("Complete the starter code below to solve the problem. Put your full solution in one "
                                            "fenced code block.")
LCB_FORMATTING_WITHOUT_STARTER_CODE = ("Read the input from standard input, solve the problem and print the answer to standard "
                                       "output. Do not run the samples. Put your full program in one fenced code block.")
CODEFORCES_SYSTEM_MESSAGE = ("You are a competitive programmer. Think about the algorithm and its complexity first, then write a "
                             "complete Python 3 program that reads standard input and writes standard output, in one fenced code block.")
