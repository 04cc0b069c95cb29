"""Shared by the GPU tests, the smoke check and the benchmark: build product layers from
oracle-quantised tensors."""
import numpy as np
import torch

from mixtral_offloading_b200 import BaseQuantizeConfig, HQQLinearTritonSavable
from oracle import hqq_oracle as O


def bf16_from_bits(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16)


def quant_config(nbits, group_size):
    return BaseQuantizeConfig(nbits=nbits, group_size=group_size, quant_zero=True, quant_scale=True)


def fill_layer(layer, od, device):
    """Point a product layer at the tensors of an oracle layer dictionary."""
    L = (od["N"] // od["group_size"]) * od["K"]
    C_ = L // od["meta_group"]
    gz = od.get("meta_group_zero") or od["meta_group"]
    Cz = L // gz
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    layer.W_q = t(od["W_q"])
    m = layer.meta
    m["scale_q"] = t(od["scale_q"]).reshape(od["meta_group"], C_)
    m["zero_q"] = t(od["zero_q"]).reshape(gz, Cz)
    m["meta_scale"]["scale"], m["meta_scale"]["zero"] = t(od["ms_scale"]).reshape(1, C_), t(od["mz_scale"]).reshape(1, C_)
    m["meta_zero"]["scale"], m["meta_zero"]["zero"] = t(od["ms_zero"]).reshape(1, Cz), t(od["mz_zero"]).reshape(1, Cz)
    layer.ready = True
    layer._desc = None
    return layer


def layer_from_oracle(od, device):
    cfg = quant_config(od["nbits"], od["group_size"])
    meta = HQQLinearTritonSavable.get_hqq_meta((od["K"], od["N"]), cfg)
    return fill_layer(HQQLinearTritonSavable(None, cfg, meta), od, device)


def random_layer(N, K, nbits, group_size, seed, std=0.02):
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn(N, K, generator=g) * std).to(torch.bfloat16)
    return O.quantize(W, nbits, group_size, 256)


def random_layer_fast(N, K, nbits, group_size, seed):
    """Random codes / scales without the float weight (for full-size shapes where only decode matters)."""
    rng = np.random.default_rng(seed)
    G = N // group_size
    L = G * K
    C_ = L // 256
    codes = rng.integers(0, 2 ** nbits, (N, K), dtype=np.uint8)
    return dict(
        N=N, K=K, nbits=nbits, group_size=group_size, meta_group=256, codes=codes, W_q=O.PACK[nbits](codes),
        scale_q=rng.integers(0, 256, L, dtype=np.uint8), zero_q=rng.integers(0, 256, L, dtype=np.uint8),
        ms_scale=(rng.uniform(0.5, 1.5, C_) * 1e-4).astype(np.float16), mz_scale=rng.uniform(-40, 0, C_).astype(np.float16),
        ms_zero=(rng.uniform(0.5, 1.5, C_) * 2e-3).astype(np.float16),
        mz_zero=rng.uniform(-700, -300, C_).astype(np.float16) if nbits == 2 else rng.uniform(-2000, -500, C_).astype(np.float16),
    )
