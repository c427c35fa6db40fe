"""Module classes with the reference's names, constructor arguments, parameter names and
``forward`` / ``shard_params`` / ``load_xsmm_params`` / ``xsmm_forward`` protocol
(src/distributed_xfold/nn/*.py), computing on the sm_100a kernels."""
from .d_triangle_multiplication import DistributeTriangleMultiplication, XSMMTriangleMultiplication  # noqa: F401
from .d_attention import DistributeGridSelfAttention  # noqa: F401
from .d_primitives import DistributeTransition, Transition, LayerNorm  # noqa: F401
from .d_diffusion_transformer import (AdaptiveLayerNorm, DistributeAdaLNZero, DistributeDiffusionTransition,  # noqa: F401
                                      DistributeSelfAttention, DistributeDiffusionTransformer)
from .d_pairformer import DistributePairformerBlock, DistributePairformerStack  # noqa: F401
