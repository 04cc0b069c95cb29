"""B200-native quantized-expert path with the module API of dvmazur/mixtral-offloading.

Importing the package does not load the CUDA library; the first operation does, and
raises if libhqq_moe_b200.so has not been built (python -m mixtral_offloading_b200.build).
"""
from .build_model import OffloadConfig, QuantConfig, make_empty_expert  # noqa: F401
from .custom_layers import (HQQLinearTritonSavable, MixtralBLockSparseTop2MLP_HQQ, ResidentMoe,  # noqa: F401
                            SparseMoeWrapper)
from .decode_model import BatchDecode, MixtralDecodeModel  # noqa: F401
from .decoder import (AttentionDecode, DecoderLayerDecode, ExpertParallelDecoderLayer, PeerExchange,  # noqa: F401
                      add_rmsnorm)
from .expert_cache import ExpertCache  # noqa: F401
from .offload_model import MixtralOffloadModel  # noqa: F401
from .expert_wrapper import MixtralExpertWrapper  # noqa: F401
from .quantize import BaseQuantizeConfig  # noqa: F401
