"""Algorithm constants shared by config validation and runtime code (reference: axon/trainer/algos/constants.py)."""

VALID_TOKEN_REDUCE = {"sum", "mean", "mean-norm", "mean-program"}
VALID_BATCH_REDUCE = {"token-mean", "step-mean", "program-mean"}
