from .manager import (CheckpointManager, CheckpointMetadata, convert_checkpoint, list_checkpoints, read_tensors, validate_checkpoint,  # noqa: F401
                      write_tensors, DTYPE_CODES)
