from fairseq2_b200.checkpoint.manager import (CheckpointError, CheckpointLoadError, CheckpointManager,
                                              CheckpointNotFoundError, CheckpointSaveError)
from fairseq2_b200.checkpoint.model_metadata import load_checkpoint_cards, save_model_metadata
