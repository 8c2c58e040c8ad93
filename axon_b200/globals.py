"""Process-wide constants (reference: axon/globals.py): debug switches read from the environment and the
delimiters reward functions use to cut a model's reasoning from its answer."""
import os

DEBUG_MOE_REPLAY = os.environ.get("DEBUG_MOE_REPLAY", "0") == "1"

# dataset preprocessing helpers that call hosted models read their names from here
GCP_PROJECT_ID = os.environ.get("GCP_PROJECT_ID", "")
GCP_LOCATION = os.environ.get("GCP_LOCATION", "us-central1")
GEMINI_MODEL = os.environ.get("GEMINI_MODEL", "gemini-1.5-pro-002")
OAI_RM_MODEL = os.environ.get("OAI_RM_MODEL", "gpt-4o-mini")

THOUGHT_DELIMITER_START = "<think>"
THOUGHT_DELIMITER_END = "</think>"
