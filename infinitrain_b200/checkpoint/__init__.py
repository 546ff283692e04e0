from .checkpoint import (Checkpoint, NewestCompleteCheckpoint, ResumeFromCheckpoint, ResumeFromCheckpointResult, SaveCheckpoint, TrainerState)
