"""Model families and their factories (public names follow the reference's
``models/__init__.py:18-125``)."""
from .kernels import (LIGER_AVAILABLE, TRITON_AVAILABLE, RMSNorm, RotaryEmbedding, MLP, Linear,
                      Embedding, rotate_half, apply_rotary_pos_emb, KernelType, create_rms_norm,
                      create_mlp, get_rotary_pos_emb_fn, create_cross_entropy_loss,
                      compute_cross_entropy_loss, FusedLinearCrossEntropy, remap_legacy_keys)
from .transformer import (TransformerModel, TransformerBlock, DenseAttention, NativeSparseAttention,
                          FlashSparseAttention, FSA_AVAILABLE, create_model)
from .mamba import (Mamba2Model, Mamba2Config, Mamba2Block, Mamba2Mixer, create_mamba2,
                    Mamba3Model, Mamba3Config, Mamba3Block, create_mamba3)
from .deltanet import (GatedDeltaNetModel, GatedDeltaNetConfig, GatedDeltaNetBlock,
                       GatedDeltaNetMixer, create_gated_deltanet)
from .hybrid import (HybridModel, HybridConfig, MambaBlock, DeltaNetBlock, AttentionBlock,
                     create_hybrid_model, get_block_classes_from_pattern, print_hybrid_model_modules)
from .configs import (get_model_config, get_mamba2_config, get_deltanet_config, get_hybrid_config,
                      get_model_type, compute_block_repeats)

__all__ = [n for n in dir() if not n.startswith("_")]
