"""B200-native TopK sparse-coder training step behind the surface of
EleutherAI/sparsify: the same exported names, computed by hand-written sm_100a
kernels (libsparsecoder.so) instead of eager PyTorch / Triton."""

__version__ = "0.1.0"

from .config import SaeConfig, SparseCoderConfig, TrainConfig, TranscoderConfig
from .fused_encoder import EncoderOutput, FusedEncoder, fused_encoder
from .sparse_coder import ForwardOutput, Sae, SparseCoder
from .trainer import SaeTrainer, Trainer

__all__ = [
    "EncoderOutput",
    "ForwardOutput",
    "FusedEncoder",
    "Sae",
    "SaeTrainer",
    "Trainer",
    "SaeConfig",
    "SparseCoder",
    "SparseCoderConfig",
    "TrainConfig",
    "TranscoderConfig",
    "fused_encoder",
]
