"""B200-native YemongPolicy trunk: masked spatial attention over ship/field tokens fused
with the per-ship Griffin RG-LRU recurrence, as hand-written sm_100a CUDA kernels behind the
reference's own ``nn.Module`` signatures.

    from boost_and_broadside_b200 import ModelConfig, ShipEncoder, TransformerBlock, YemongBlock, YemongTrunk

The modules mirror ``boost_and_broadside.models.yemong.{attention,griffin}`` of the
reference (same constructor arguments, parameter names and forward signatures) and call
the C-ABI library ``libbnb_trunk.so`` (include/bnb_trunk.h).  There is no CPU path.
"""

from .config import ModelConfig
from .yemong.attention import GatedMLP, TransformerBlock
from .yemong.encoder import BulletEncoder, ShipEncoder
from .yemong.heads import HeadMLP, NextStateHead, TeamPMA, evaluate_action, sample_action
from .yemong.griffin import CONV_KERNEL, RGLRU, GriffinTemporalBlock, YemongBlock
from .yemong.policy import YemongPolicy
from .yemong.trunk import YemongTrunk, RaggedBatch

__all__ = [
    "BulletEncoder",
    "CONV_KERNEL",
    "GatedMLP",
    "GriffinTemporalBlock",
    "HeadMLP",
    "ModelConfig",
    "NextStateHead",
    "RGLRU",
    "RaggedBatch",
    "ShipEncoder",
    "TeamPMA",
    "TransformerBlock",
    "YemongBlock",
    "YemongPolicy",
    "YemongTrunk",
    "evaluate_action",
    "sample_action",
]
