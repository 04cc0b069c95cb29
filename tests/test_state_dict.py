"""State-dict (de)serialisation of the quantized layer and of the expert slab: the keys and the round trip the
reference's hooks define (src/custom_layers.py:136-222, src/expert_wrapper.py:23-30).  Runs on the CPU: the hooks
only move tensors."""
import numpy as np
import torch

from mixtral_offloading_b200 import HQQLinearTritonSavable
from tests.helpers import fill_layer, quant_config, random_layer

REFERENCE_KEYS = {"W_q", "meta.scale_q", "meta.meta_scale.scale", "meta.meta_scale.zero", "meta.zero_q",
                  "meta.meta_zero.scale", "meta.meta_zero.zero"}          # custom_layers.py:147-164


def _layer(od, device="cpu"):
    cfg = quant_config(od["nbits"], od["group_size"])
    meta = HQQLinearTritonSavable.get_hqq_meta((od["K"], od["N"]), cfg)
    return fill_layer(HQQLinearTritonSavable(None, cfg, meta), od, device)


def test_state_dict_keys_and_round_trip():
    od = random_layer(128, 256, 4, 64, seed=3)
    src = _layer(od)
    sd = src.state_dict()
    assert set(sd) == REFERENCE_KEYS
    dst = HQQLinearTritonSavable(None, quant_config(4, 64), HQQLinearTritonSavable.get_hqq_meta((256, 128), quant_config(4, 64)))
    assert not dst.ready
    dst.load_state_dict(sd)
    assert dst.ready and set(dst.state_dict()) == REFERENCE_KEYS
    for k, v in sd.items():
        assert torch.equal(dst.state_dict()[k], v), k
    assert np.array_equal(dst.W_q.numpy(), od["W_q"])


def test_bias_travels_and_becomes_bf16():
    od = random_layer(128, 256, 2, 16, seed=4)
    src = _layer(od)
    src.bias = torch.randn(128).to(torch.float16)                         # the reference's layers are fp16
    sd = src.state_dict()
    assert "bias" in sd
    dst = _layer(random_layer(128, 256, 2, 16, seed=5))
    dst.load_state_dict(sd)
    assert dst.bias.dtype == torch.bfloat16
    assert torch.equal(dst.bias, sd["bias"].to(torch.bfloat16))


def test_nested_module_prefixes():
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = _layer(random_layer(64, 128, 4, 32, seed=6))
            self.k_proj = _layer(random_layer(64, 128, 4, 32, seed=7))
    a, b = Block(), Block()
    sd = a.state_dict()
    assert {"q_proj." + k for k in REFERENCE_KEYS} | {"k_proj." + k for k in REFERENCE_KEYS} == set(sd)
    b.load_state_dict(sd)
    for k, v in sd.items():
        assert torch.equal(b.state_dict()[k], v), k
