from fairseq2_b200.nn.batch_layout import BatchLayout
from fairseq2_b200.nn.embedding import (Embedding, ShardedEmbedding, StandardEmbedding, VocabShardedEmbedding,
                                        init_scaled_embedding)
from fairseq2_b200.nn.incremental_state import IncrementalState, IncrementalStateBag
from fairseq2_b200.nn.normalization import LayerNorm, RMSNorm, StandardLayerNorm
from fairseq2_b200.nn.position_encoder import (DualRotaryEncoder, LearnedPositionEncoder, PositionEncoder,
                                               ReferenceRotaryEncoder,
                                               RotaryEncoder, SinusoidalPositionEncoder)
from fairseq2_b200.nn.projection import (ColumnShardedLinear, IdentityProjection, Linear, Projection,
                                         RowShardedLinear, TiedProjection)
from fairseq2_b200.nn.residual import (AdditiveResidualConnect, DropPathResidualConnect, ResidualConnect,
                                       ScaledResidualConnect)
from fairseq2_b200.nn.sharded import Sharded, get_shard_dims
