"""Configuration objects of the reference's src/build_model.py (OffloadConfig :30-35,
QuantConfig :38-52) and the expert constructors it calls (:123-134).  Loading a
checkpoint from the Hugging Face hub is outside this package's scope; the tests and
the benchmark build random-initialised models through these same constructors.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import cache

from .custom_layers import HQQLinearTritonSavable, MixtralBLockSparseTop2MLP_HQQ


@dataclass(frozen=True)
class OffloadConfig:
    main_size: int
    offload_size: int
    buffer_size: int
    offload_per_layer: int


class QuantConfig:
    def __init__(self, ffn_config, attn_config):
        self.ffn_config = ffn_config
        self.attn_config = attn_config

    @cache
    def get_ffn_metas(self, hidden_dim: int, ffn_dim: int):
        return (
            HQQLinearTritonSavable.get_hqq_meta((hidden_dim, ffn_dim), self.ffn_config),
            HQQLinearTritonSavable.get_hqq_meta((ffn_dim, hidden_dim), self.ffn_config),
        )


def make_empty_expert(model_config, quant_config: QuantConfig) -> MixtralBLockSparseTop2MLP_HQQ:
    """build_model.py:123-134."""
    meta1, meta2 = quant_config.get_ffn_metas(model_config.hidden_size, model_config.intermediate_size)
    return MixtralBLockSparseTop2MLP_HQQ(model_config, quant_config.ffn_config, meta1, meta2)
