"""Stand-in for the `hqq` import surface, used ONLY by make_golden.py.

The reference's files import `hqq.core.quantize` (HQQLinear, Quantizer,
BaseQuantizeConfig) and `hqq.core.bitpack` (BitPack).  hqq (pinned at
37502bea31f2969c6680c0c4a88ca74b3bb234a5 in the reference's requirements.txt)
is not installed and cannot be fetched, so this module registers a minimal
replacement in sys.modules before the reference is imported.  What it defines
is this build's own quantiser (min/max affine, round to nearest, groups along
axis 0, 8-bit scale/zero in groups of 256); everything downstream of it —
packing, repack, dequantize, the expert FFN, the MoE block, the cache — is the
reference's unmodified code.
"""
from __future__ import annotations

import importlib.machinery
import sys
import types

import torch
from torch import nn


class Quantizer:
    pack = {"8bit_u8": lambda t: t.to(torch.uint8)}
    unpack = {"8bit_u8": lambda t: t}
    bit_to_packing = {8: "8bit_u8", 4: "4bit_u8", 3: "3bit_32", 2: "2bit_u8"}

    @classmethod
    def quantize(cls, tensor, nbits=4, channel_wise=True, group_size=64, optimize=False,
                 round_zero=False, axis=0):
        assert axis == 0 and channel_wise and group_size is not None
        shape = tensor.shape
        v = tensor.detach().to(torch.float32).reshape(group_size, -1)
        vmin = v.min(dim=0, keepdim=True).values
        vmax = v.max(dim=0, keepdim=True).values
        qmax = float(2 ** nbits - 1)
        q_scale = (qmax / (vmax - vmin)).clamp(max=2e4)
        zero = -vmin * q_scale
        codes = torch.round(v * q_scale + zero).clamp(0, qmax).to(torch.uint8)
        packing = cls.bit_to_packing[nbits]
        meta = {"nbits": nbits, "group_size": group_size, "shape": shape, "scale": 1.0 / q_scale,
                "zero": zero, "axis": axis, "packing": packing}
        return cls.pack[packing](codes), meta

    @classmethod
    def dequantize(cls, W_q, meta):
        q = cls.unpack[meta["packing"]](W_q).half()
        if meta["group_size"] is not None and meta["nbits"] == 3:
            q = q[: meta["group_size"]]
        return ((q - meta["zero"]) * meta["scale"]).reshape(meta["shape"])


class BitPack:
    """Only reached through the reference's *_universal fallbacks for untagged tensors."""
    unpack_4bit_u8 = unpack_2bit_u8 = unpack_3bit_32 = None


def BaseQuantizeConfig(nbits=4, group_size=64, quant_zero=True, quant_scale=False):
    meta_q = {"nbits": 8, "channel_wise": True, "group_size": 256, "optimize": False}
    return {
        "weight_quant_params": {"nbits": nbits, "channel_wise": True, "group_size": group_size,
                                "optimize": False, "round_zero": False},
        "scale_quant_params": dict(meta_q) if quant_scale else None,
        "zero_quant_params": dict(meta_q) if quant_zero else None,
    }


class HQQLinear(nn.Module):
    def __init__(self, linear_layer, quant_config, del_orig=True, compute_dtype=torch.float16):
        super().__init__()
        self.ready = False
        self.in_gpu = False
        self.quant_config = quant_config
        self.bias = None
        if linear_layer is not None:
            self.bias = None if linear_layer.bias is None else linear_layer.bias.half()
            self.quantize(linear_layer.weight.data, **quant_config)

    def quantize(self, W, weight_quant_params, scale_quant_params, zero_quant_params):
        W_q, meta = Quantizer.quantize(W, **weight_quant_params)
        meta["quant_scale"] = scale_quant_params is not None
        meta["quant_zero"] = zero_quant_params is not None
        for name, params in (("scale", scale_quant_params), ("zero", zero_quant_params)):
            if params is None:
                meta[name] = meta[name].half()
                continue
            q, m = Quantizer.quantize(meta[name], **params)
            m["scale"], m["zero"] = m["scale"].half(), m["zero"].half()
            meta[name + "_q"], meta["meta_" + name] = q, m
            del meta[name]
        self.W_q, self.meta, self.ready = W_q, meta, True


def install():
    """Register the stand-in modules (with a spec, or transformers' hqq probe fails)."""
    # transformers probes for hqq while these import; they must be loaded before the stand-in exists
    import transformers.activations  # noqa: F401
    import transformers.cache_utils  # noqa: F401
    import transformers.models.mixtral.configuration_mixtral  # noqa: F401

    def mod(name):
        m = types.ModuleType(name)
        m.__spec__ = importlib.machinery.ModuleSpec(name, None)
        sys.modules[name] = m
        return m

    hqq, core, quant, bitpack = mod("hqq"), mod("hqq.core"), mod("hqq.core.quantize"), mod("hqq.core.bitpack")
    hqq.core, core.quantize, core.bitpack = core, quant, bitpack
    quant.Quantizer, quant.HQQLinear, quant.BaseQuantizeConfig = Quantizer, HQQLinear, BaseQuantizeConfig
    bitpack.BitPack = BitPack
