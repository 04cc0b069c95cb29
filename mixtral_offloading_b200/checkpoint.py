"""Checkpoints in the reference's on-disk layout, and a loader that builds a decoder from one without the hub.

The reference's build_model (src/build_model.py:137-241) reads a directory with
  model.safetensors.index.json   {"weight_map": {tensor name: file name}}
  one file for the trunk         embeddings, norms, gates, lm_head and the quantized attention projections
                                 (found through weight_map["model.embed_tokens.weight"], :194-202)
  one file per expert            model.layers.{l}.block_sparse_moe.experts.{e}.w{1,2,3}.{W_q, meta.*}
                                 (found through ...experts.{e}.w1.W_q, :146-151; loaded with strict=True into an
                                 empty MixtralBLockSparseTop2MLP_HQQ whose hooks take the tensors, :152-153)
with Hugging Face Mixtral parameter names.  The model's dimensions come from the hub there
(AutoConfig.from_pretrained, :172-184); here the directory also carries them in hqm_config.json, so that no
network is needed.  Tensors are stored in the layout the layers hold in memory: W_q (N/per, K) as repack() leaves
it.  (Files written by the reference's own quantisation script hold hqq's stock bit layout instead; hqq is needed
to read those.)

  save_checkpoint(dir, ...)      writes such a directory from live modules
  load_expert(dir, ...)          make_and_load_expert_wrapper, build_model.py:137-155
  load_decode_model(dir, ...)    the resident-expert decoder (MixtralDecodeModel) from a directory
  build_model(device, quant_config, offload_config, dir)
                                 build_model.py:166-241: the decoder with offloaded experts (MixtralOffloadModel)
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import torch
from safetensors.torch import load_file, save_file

from .build_model import OffloadConfig, QuantConfig, make_empty_expert
from .custom_layers import HQQLinearTritonSavable, ResidentMoe, SparseMoeWrapper
from .decode_model import MixtralDecodeModel
from .decoder import AttentionDecode, DecoderLayerDecode
from .expert_cache import ExpertCache
from .expert_wrapper import MixtralExpertWrapper
from .offload_model import MixtralOffloadModel
from .quantize import BaseQuantizeConfig

INDEX = "model.safetensors.index.json"
CONFIG = "hqm_config.json"
TRUNK_FILE = "trunk.safetensors"


def expert_prefix(layer: int, expert: int) -> str:
    return f"model.layers.{layer}.block_sparse_moe.experts.{expert}"       # build_model.py:148


def expert_file(layer: int, expert: int) -> str:
    return f"layer_{layer}_expert_{expert}.safetensors"


class ModelConfig:
    """The fields of MixtralConfig this path reads (build_model.py:123-134, custom_layers.py:259-270)."""

    def __init__(self, d: dict):
        self.hidden_size, self.intermediate_size = int(d["hidden_size"]), int(d["intermediate_size"])
        self.num_hidden_layers, self.vocab_size = int(d["num_hidden_layers"]), int(d["vocab_size"])
        self.num_attention_heads, self.num_key_value_heads = int(d["num_attention_heads"]), int(d["num_key_value_heads"])
        self.head_dim = int(d.get("head_dim", self.hidden_size // self.num_attention_heads))
        self.num_local_experts, self.num_experts_per_tok = int(d["num_local_experts"]), int(d.get("num_experts_per_tok", 2))
        self.rope_theta, self.rms_norm_eps = float(d.get("rope_theta", 1e6)), float(d.get("rms_norm_eps", 1e-5))
        self.hidden_act = d.get("hidden_act", "silu")
        self.attn_quant, self.ffn_quant = d["attn_quant"], d["ffn_quant"]     # {"nbits": .., "group_size": ..}

    def quant_config(self) -> QuantConfig:
        mk = lambda q: BaseQuantizeConfig(nbits=int(q["nbits"]), group_size=int(q["group_size"]), quant_zero=True, quant_scale=True)
        return QuantConfig(ffn_config=mk(self.ffn_quant), attn_config=mk(self.attn_quant))


def _layer_state(prefix: str, layer: HQQLinearTritonSavable) -> Dict[str, torch.Tensor]:
    return {f"{prefix}.{k}": v.detach().cpu().contiguous() for k, v in layer.state_dict().items()}


def save_checkpoint(states_dir: str, config: dict, embed: torch.Tensor, lm_head: torch.Tensor, final_norm: torch.Tensor,
                    layers: Sequence[dict]) -> None:
    """layers[l] = {"q","k","v","o": HQQLinearTritonSavable, "ln_in","ln_post": (hidden) tensors,
    "gate": (E, hidden) tensor, "experts": [MixtralBLockSparseTop2MLP_HQQ or MixtralExpertWrapper, ...]}."""
    os.makedirs(states_dir, exist_ok=True)
    weight_map: Dict[str, str] = {}
    trunk = {"model.embed_tokens.weight": embed, "model.norm.weight": final_norm, "lm_head.weight": lm_head}
    for l, ly in enumerate(layers):
        base = f"model.layers.{l}"
        trunk[f"{base}.input_layernorm.weight"] = ly["ln_in"]
        trunk[f"{base}.post_attention_layernorm.weight"] = ly["ln_post"]
        trunk[f"{base}.block_sparse_moe.gate.weight"] = ly["gate"]
        for name in ("q", "k", "v", "o"):
            trunk.update(_layer_state(f"{base}.self_attn.{name}_proj", ly[name]))
        for e, expert in enumerate(ly["experts"]):
            ffn = ResidentMoe._ffn(expert)
            state = {}
            for w in ("w1", "w2", "w3"):
                state.update(_layer_state(f"{expert_prefix(l, e)}.{w}", getattr(ffn, w)))
            save_file(state, os.path.join(states_dir, expert_file(l, e)))
            weight_map.update({k: expert_file(l, e) for k in state})
    trunk = {k: v.detach().cpu().contiguous() for k, v in trunk.items()}
    save_file(trunk, os.path.join(states_dir, TRUNK_FILE))
    weight_map.update({k: TRUNK_FILE for k in trunk})
    with open(os.path.join(states_dir, INDEX), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    with open(os.path.join(states_dir, CONFIG), "w") as f:
        json.dump(config, f)


def _weight_map(states_dir: str) -> Dict[str, str]:
    with open(os.path.join(states_dir, INDEX)) as f:
        return json.load(f)["weight_map"]


def load_config(states_dir: str) -> ModelConfig:
    with open(os.path.join(states_dir, CONFIG)) as f:
        return ModelConfig(json.load(f))


def load_expert(states_dir: str, config: ModelConfig, quant_config: QuantConfig, expert_uid, device) -> MixtralExpertWrapper:
    """make_and_load_expert_wrapper (build_model.py:137-155): the expert's file is found through the index entry of
    its w1.W_q, loaded strictly into an empty expert, wrapped into one slab."""
    layer_idx, expert_idx = expert_uid
    prefix = expert_prefix(layer_idx, expert_idx)
    fname = _weight_map(states_dir)[f"{prefix}.w1.W_q"]
    state = load_file(os.path.join(states_dir, fname), device=str(device))
    state = {k[len(prefix) + 1:]: v for k, v in state.items() if k.startswith(prefix + ".")}
    expert = make_empty_expert(config, quant_config)
    expert.load_state_dict(state, strict=True)
    return MixtralExpertWrapper(expert, device)


def _load_linear(trunk: Dict[str, torch.Tensor], prefix: str, shape, quant) -> HQQLinearTritonSavable:
    layer = HQQLinearTritonSavable(None, quant, HQQLinearTritonSavable.get_hqq_meta(shape, quant))
    layer.load_state_dict({k[len(prefix) + 1:]: v for k, v in trunk.items() if k.startswith(prefix + ".")}, strict=True)
    return layer


def _bf(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).contiguous()


def _load_trunk(states_dir: str, device):
    wm = _weight_map(states_dir)
    return load_file(os.path.join(states_dir, wm["model.embed_tokens.weight"]), device=str(device))   # build_model.py:194-202


def _load_attention(trunk, cfg: ModelConfig, qc: QuantConfig, l: int, max_len: int) -> AttentionDecode:
    """The layer's four quantized projections (replace_attn_layers, build_model.py:55-120) and its two norms."""
    H, nh, nkv, hd = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    base = f"model.layers.{l}"
    proj = {n: _load_linear(trunk, f"{base}.self_attn.{n}_proj", shape, qc.attn_config)
            for n, shape in (("q", (H, nh * hd)), ("k", (H, nkv * hd)), ("v", (H, nkv * hd)), ("o", (nh * hd, H)))}
    return AttentionDecode(proj["q"], proj["k"], proj["v"], proj["o"], _bf(trunk[f"{base}.input_layernorm.weight"]),
                           _bf(trunk[f"{base}.post_attention_layernorm.weight"]), nh, nkv, hd, max_len,
                           rope_theta=cfg.rope_theta, rms_eps=cfg.rms_norm_eps)


def _load_gate(trunk, cfg: ModelConfig, l: int, device) -> torch.nn.Linear:
    gate = torch.nn.Linear(cfg.hidden_size, cfg.num_local_experts, bias=False, dtype=torch.bfloat16, device=device)
    gate.weight.data = _bf(trunk[f"model.layers.{l}.block_sparse_moe.gate.weight"])
    return gate


def build_model(device, quant_config, offload_config: OffloadConfig, state_path: str, max_len: int = 4096,
                speculate: bool = False) -> MixtralOffloadModel:
    """build_model.py:166-241: one ExpertCache of offload_config's sizes over all layers, each layer its own eviction
    group, the first offload_per_layer experts of every layer placed in host memory (:224), SparseMoeWrapper in every
    layer.  quant_config=None takes the quantisation recorded in the directory.  The slabs' template is expert (0, 0),
    as in the reference (:157-163, :176-180)."""
    device = torch.device(device)
    cfg = load_config(state_path)
    qc = quant_config if quant_config is not None else cfg.quant_config()
    trunk = _load_trunk(state_path, device)

    def _make_module():
        return load_expert(state_path, cfg, qc, (0, 0), device)
    cache = ExpertCache(make_module=_make_module, main_size=offload_config.main_size,
                        offload_size=offload_config.offload_size, buffer_size=offload_config.buffer_size)
    attentions, blocks = [], []
    for l in range(cfg.num_hidden_layers):
        attentions.append(_load_attention(trunk, cfg, qc, l, max_len))
        blocks.append(SparseMoeWrapper(cfg, l, _load_gate(trunk, cfg, l, device), cache))
        for e in range(cfg.num_local_experts):
            wrapper = load_expert(state_path, cfg, qc, (l, e), device)
            cache.add_expert(uid=(l, e), module=wrapper, eviction_group=l, offload=e < offload_config.offload_per_layer)
            del wrapper
    return MixtralOffloadModel(_bf(trunk["model.embed_tokens.weight"]), attentions, blocks, _bf(trunk["model.norm.weight"]),
                               _bf(trunk["lm_head.weight"]), rms_eps=cfg.rms_norm_eps, speculate=speculate)


def load_decode_model(states_dir: str, device, max_len: int) -> MixtralDecodeModel:
    """Every expert resident on `device`: the decoder build_model.py:166-241 would assemble around Hugging Face's
    MixtralForCausalLM, as this package's own decode model."""
    cfg = load_config(states_dir)
    qc = cfg.quant_config()
    trunk = _load_trunk(states_dir, device)
    bf = _bf
    lns_in = [bf(trunk[f"model.layers.{l}.input_layernorm.weight"]) for l in range(cfg.num_hidden_layers)]
    final_norm = bf(trunk["model.norm.weight"])
    layers: List[DecoderLayerDecode] = []
    for l in range(cfg.num_hidden_layers):
        attn = _load_attention(trunk, cfg, qc, l, max_len)
        gate = _load_gate(trunk, cfg, l, device)
        experts = [load_expert(states_dir, cfg, qc, (l, e), device) for e in range(cfg.num_local_experts)]
        moe = ResidentMoe(cfg, l, gate, experts)
        next_ln = lns_in[l + 1] if l + 1 < cfg.num_hidden_layers else final_norm
        layers.append(DecoderLayerDecode(attn, moe, next_ln))
    return MixtralDecodeModel(bf(trunk["model.embed_tokens.weight"]), layers, lns_in[0], bf(trunk["lm_head.weight"]),
                              rms_eps=cfg.rms_norm_eps)
