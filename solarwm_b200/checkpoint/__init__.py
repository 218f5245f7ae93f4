"""Atomic checkpoint directories with a size-inventory manifest (layout ``solarwm.checkpoint.v2``)."""
from .store import (CheckpointContract, CheckpointTransaction, ComponentFile, VerifiedCheckpoint,  # noqa: F401
                    assert_resume_compatible, verify_checkpoint)
