"""The quantiser that produces codes / scale / zero for a layer.

In the reference this role is played by the third-party hqq package
(BaseQuantizeConfig, Quantizer.quantize as called from src/custom_layers.py:26,36
and src/build_model.py:110); hqq is not part of the reference tree, so the
quantiser here is this package's own: min/max affine, round to nearest, groups of
`group_size` along axis 0 of the (group_size, -1) view, and the resulting scale and
zero vectors quantised once more to 8 bit in groups of 256 the same way.  It runs
at model-build time only and is plain torch; the per-token path never calls it.
"""
from __future__ import annotations

import torch

META_GROUP = 256


def BaseQuantizeConfig(nbits: int = 4, group_size: int = 64, quant_zero: bool = True, quant_scale: bool = False):
    """Same call and same dictionary keys as hqq's BaseQuantizeConfig as the reference uses it
    (notebooks/demo.ipynb:1220-1235, src/custom_layers.py:24)."""
    meta_q = {"nbits": 8, "channel_wise": True, "group_size": META_GROUP, "optimize": False}
    return {
        "weight_quant_params": {"nbits": nbits, "channel_wise": True, "group_size": group_size,
                                "optimize": False, "round_zero": False},
        "scale_quant_params": dict(meta_q) if quant_scale else None,
        "zero_quant_params": dict(meta_q) if quant_zero else None,
    }


def affine_quantize(t: torch.Tensor, nbits: int, group_size: int):
    """codes (group_size, -1) uint8 and the dequantisation (scale, zero), each (1, -1) fp32:
    value ~= (code - zero) * scale."""
    v = t.detach().to(torch.float32).reshape(group_size, -1)
    vmin = v.min(dim=0, keepdim=True).values
    vmax = v.max(dim=0, keepdim=True).values
    qmax = float(2 ** nbits - 1)
    q_scale = (qmax / (vmax - vmin)).clamp(max=2e4)
    zero = -vmin * q_scale
    codes = torch.round(v * q_scale + zero).clamp(0, qmax).to(torch.uint8)
    return codes, 1.0 / q_scale, zero


def meta_template(shape, quant_config) -> dict:
    """The non-tensor part of a layer's meta (what get_hqq_meta returns, custom_layers.py:118-134)."""
    wq = quant_config["weight_quant_params"]
    N, K = int(shape[0]), int(shape[1])
    nbits, g = int(wq["nbits"]), int(wq["group_size"])
    assert N % g == 0, f"out_features {N} must be a multiple of group_size {g}"
    L = (N // g) * K
    meta = {"nbits": nbits, "group_size": g, "shape": torch.Size((N, K)), "axis": 0,
            "packing": {4: "4bit_u8", 3: "3bit_32", 2: "2bit_u8"}[nbits],
            "quant_scale": quant_config.get("scale_quant_params") is not None,
            "quant_zero": quant_config.get("zero_quant_params") is not None}
    for name in ("scale", "zero"):
        params = quant_config.get(name + "_quant_params")
        if params is not None:
            mg = int(params["group_size"])
            assert int(params["nbits"]) == 8 and L % mg == 0
            meta["meta_" + name] = {"nbits": 8, "group_size": mg, "shape": torch.Size((1, L)), "axis": 0,
                                    "packing": "8bit_u8"}
    return meta
