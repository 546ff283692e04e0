from .checkpoint import (Checkpoint, ResumeFromCheckpoint, ResumeFromCheckpointResult, SaveCheckpoint, TrainerState)
