from fairseq2_b200.optim.adafactor import Adafactor
from fairseq2_b200.optim.adamw import AdamW
from fairseq2_b200.optim.fp16_loss_scaler import (Float16LossScaler, Float16LossScaleResult, NoopFloat16LossScaler,
                                                  StandardFloat16LossScaler)
from fairseq2_b200.optim.lr_schedulers import (AbstractLRScheduler, CosineAnnealingLR, MyleLR, NoamLR, NoopLR,
                                               PassthroughLR, PolynomialDecayLR, TriStageLR, get_effective_lr)
