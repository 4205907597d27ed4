from fairseq2_b200.model_checkpoint.common import reshard_tensor
from fairseq2_b200.model_checkpoint.loader import (BasicModelCheckpointLoader, DelegatingModelCheckpointLoader,
                                                   LLaMAModelCheckpointLoader, ModelCheckpointError,
                                                   ModelCheckpointLoader, NativeModelCheckpointLoader,
                                                   SafetensorsCheckpointLoader, create_default_checkpoint_loader)
