"""Parts a layer is put together from, and their registries."""
from .attention import GQAttention
from .base import (FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, StepBatch, StepContext, WeightSpec,
                   float32_vector)
from .block import ParallelResidualBlock, PostnormResidualBlock, PrenormResidualBlock
from .decayed_state import DecayedStateMixer
from .delta_rule import DeltaRuleMixer
from .embedding import LMHead, TokenEmbedding
from .feed_forward import SwiGLU
from .gated_delta import GatedDeltaMixer
from .latent_attention import LatentAttention
from .mlstm import MatrixMemoryMixer
from .norm import GroupRMSNorm, RMSNorm
from .position import RotaryHalved, RotaryTables
from .side_by_side import SideBySideMixer
from .sigmoid_attention import SigmoidAttention
from .state_space import StateSpaceMixer
from .residual_streams import ResidualStreams, StreamConnection, StreamsBlock
from .routed_experts import TableExperts
from .softmax_attention import SoftmaxAttention
from .registry import make_block, make_part, part_kinds, register_block, register_part, unregister_part

register_part("rms_norm", RMSNorm, replace=True)
register_part("group_rms_norm", GroupRMSNorm, replace=True)
register_part("delta_rule_mixer", DeltaRuleMixer, replace=True)
register_part("decayed_state_mixer", DecayedStateMixer, replace=True)
register_part("sigmoid_attention", SigmoidAttention, replace=True)
register_part("side_by_side", SideBySideMixer, replace=True)
register_part("rotary_halved", RotaryHalved, replace=True)
register_part("rotary_tables", RotaryTables, replace=True)
register_part("latent_attention", LatentAttention, replace=True)
register_part("state_space_mixer", StateSpaceMixer, replace=True)
register_part("gated_delta_mixer", GatedDeltaMixer, replace=True)
register_part("gqa_attention", GQAttention, replace=True)
register_part("softmax_attention", SoftmaxAttention, replace=True)
register_part("table_experts", TableExperts, replace=True)
register_part("routed_experts", TableExperts, replace=True)
register_part("mlstm_mixer", MatrixMemoryMixer, replace=True)
register_part("stream_connection", StreamConnection, replace=True)
register_part("swiglu", SwiGLU, replace=True)
register_part("token_embedding", TokenEmbedding, replace=True)
register_part("lm_head", LMHead, replace=True)
register_block("prenorm_residual", PrenormResidualBlock, replace=True)
register_block("parallel_residual", ParallelResidualBlock, replace=True)
register_block("residual_streams", StreamsBlock, replace=True)
register_block("postnorm_residual", PostnormResidualBlock, replace=True)

__all__ = ["MatrixMemoryMixer", "PostnormResidualBlock", "ResidualStreams", "SoftmaxAttention", "StreamConnection", "StreamsBlock", "TableExperts", "GatedDeltaMixer", "LatentAttention", "ParallelResidualBlock", "RotaryTables", "StateSpaceMixer", "DecayedStateMixer", "DeltaRuleMixer", "GroupRMSNorm", "SideBySideMixer", "SigmoidAttention",
           "FeedForward", "GQAttention", "LMHead", "Mixer", "Norm", "Part", "PositionEncoding",
           "PrenormResidualBlock", "RMSNorm", "RotaryHalved", "Runtime", "StepBatch", "StepContext", "SwiGLU",
           "TokenEmbedding", "WeightSpec", "float32_vector", "make_block", "make_part", "part_kinds",
           "register_block", "register_part", "unregister_part"]
