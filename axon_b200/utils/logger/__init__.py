from .aggregate_logger import (DecoratorLoggerBase, LocalLogger, concat_dict_to_str, log_with_rank, print_rank_0,  # noqa: F401
                               print_with_rank, print_with_rank_and_timer)
