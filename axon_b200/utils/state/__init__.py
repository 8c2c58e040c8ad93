from .state_manager import BaseStateManager, StateSaveMode
from .fsdp_state_manager import FSDPStateManager
from .utils import (delete_oldest_checkpoints, find_latest_ckpt_path, get_checkpoint_directories, is_valid_checkpoint)

__all__ = ["BaseStateManager", "StateSaveMode", "FSDPStateManager", "delete_oldest_checkpoints",
           "find_latest_ckpt_path", "get_checkpoint_directories", "is_valid_checkpoint"]
