from .checkpoint import (AsyncCheckpointWriter, build_checkpoint, load_checkpoint,
                         model_from_checkpoint, save_checkpoint)

__all__ = ["AsyncCheckpointWriter", "build_checkpoint", "load_checkpoint", "model_from_checkpoint",
           "save_checkpoint"]
