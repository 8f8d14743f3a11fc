"""Pogorax: a pre-norm decoder on an fp32 residual stream whose token mixers are, in any order, (a) a PAIR of softmax
attention without positions, masked to blocks of positions, with a sigmoid output gate, beside a matrix memory with
exponential gates; (b) a PAIR of causal softmax attention with interleaved rotary positions on a part of every head and
unit-RMS q / k, beside a real-gated linear recurrent unit; (c) a selective state space.  A pair's two outputs are each
RMS-normed over the model width and averaged.  Feed-forwards are gated (tanh-GELU) or absent; the embedding is scaled.

The model is the generic backbone (`transformer.py`) configured by `ModelConfig.layer_specs`; this module only reads the
family's `config.json` / tensor names.  A checkpoint is `config.json` + `model.safetensors` with

    embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.mlp.{gate,up,down},
    l<i>.mix.<name> (selective state space), l<i>.mix.{left,right}.<name> and l<i>.mix.{left,right}.out (pairs)

Which options an attention part carries is read from what the checkpoint holds: `rot` / `mask` entries of its config, a
gate matrix among its tensors.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from .config import LayerSpec, MixerSpec, ModelConfig
from .gopunex import read_safetensors_shapes
from .transformer import TransformerLMHeadModel

__all__ = ["PogoraxForCausalLM", "pogorax_config", "convert_pogorax_state_dict", "load_pogorax"]

# what the design fixes for its mixers
_PAIR_RIGHT = {"parallel": "mlstm", "parallel_2": "rglru"}
_LRU_C = 8.0


class PogoraxForCausalLM(TransformerLMHeadModel):
    pass


def _attention_spec(m: dict, unit_norm: bool, gated: bool) -> MixerSpec:
    rot, mask = m.get("rot") or {}, m.get("mask") or {}
    return MixerSpec(kind="attention", heads=m["heads"], kv_heads=m.get("kv_heads", m["heads"]), dim=m["dim"],
                     vdim=m.get("vdim", m["dim"]), scale=m["scale"], rot_dims=int(rot.get("dims", 0)),
                     rot_base=float(rot.get("base", 10000.0)), rot_interleaved=True, head_unit_norm=unit_norm,
                     mask_block=int(mask.get("size", 0)), out_gate=gated, wide_weights=True)


def pogorax_config(hf: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> ModelConfig:
    shapes = shapes or {}
    specs = []
    for i, ly in enumerate(hf["layers"]):
        m, kind = ly["mixer"], ly["type"]
        if kind == "mamba2":
            mixer = MixerSpec(kind="ssd", heads=m["heads"], vdim=m["vdim"], dim=m["state"], state=m["state"],
                              groups=m.get("groups", 1), norm_groups=m.get("norm_groups", 1), conv=m["conv"])
        elif kind in _PAIR_RIGHT:
            lm, rm = m["left"], m["right"]
            # the first pair's attention is gated and unrotated, the second's rotated with unit-RMS heads; a gate matrix
            # among the tensors (when the shapes are known) decides the gate
            gated = (f"l{i}.mix.left.g" in shapes) if shapes else kind == "parallel"
            left = _attention_spec(lm, unit_norm=kind == "parallel_2", gated=gated)
            if _PAIR_RIGHT[kind] == "mlstm":
                right = MixerSpec(kind="mlstm", heads=rm["heads"], dim=rm["dim"], vdim=rm.get("vdim", rm["dim"]),
                                  gate_cap=float(rm.get("gate_cap", 0.0)))
            else:
                right = MixerSpec(kind="rglru", lru_width=rm["width"], blocks=rm.get("blocks", 1), conv=rm["conv"],
                                  lru_c=_LRU_C)
            mixer = MixerSpec(kind="pair", parts=[left, right])
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = ly.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        specs.append(LayerSpec(mixer=mixer, ff=None if mlp is None else mlp["ff"]))
    ffs = [s.ff for s in specs if s.ff is not None]
    return ModelConfig(model_type="pogorax", vocab_size=hf["vocab"], hidden_size=hf["width"],
                       intermediate_size=max(ffs) if ffs else hf["width"], layer_specs=specs,
                       norm_eps=hf["norm"]["eps"], norm_type="rms", hidden_act="gelu_tanh", glu=True, pos_type="none",
                       embed_scale=hf.get("embedding", {}).get("scale", 1.0), fp32_residual=True, fp32_logits=True,
                       tie_word_embeddings=False, max_position_embeddings=1 << 20)


def _convert_mixer(sd: Dict[str, torch.Tensor], m: str, a: str, mx: MixerSpec, out: Dict[str, torch.Tensor]) -> None:
    """Tensors `m + name` of one mixer -> parameters `a + name`; projections that read the same input are stacked."""
    if mx.kind == "attention":
        rows = [sd[m + "q"], sd[m + "k"], sd[m + "v"]] + ([sd[m + "g"]] if mx.out_gate else [])
        out[a + "qkv_proj.weight"] = torch.cat(rows, 0)
    elif mx.kind == "mlstm":
        out[a + "in_proj.weight"] = torch.cat([sd[m + n] for n in ("q", "k", "v", "g", "i", "f")], 0)
        out[a + "gate_bias"] = torch.cat([sd[m + "i.b"], sd[m + "f.b"]], 0)
        out[a + "norm_weight"] = sd[m + "norm"]
    elif mx.kind == "rglru":
        out[a + "in_proj.weight"] = torch.cat([sd[m + "y"], sd[m + "x"]], 0)
        out[a + "in_proj.bias"] = torch.cat([sd[m + "y.b"], sd[m + "x.b"]], 0)
        out[a + "conv_weight"], out[a + "conv_bias"] = sd[m + "conv"], sd[m + "conv.b"]
        out[a + "gate_weight"] = torch.cat([sd[m + "ra"], sd[m + "ri"]], 1)           # [blocks, 2 bw (out), bw (in)]
        out[a + "gate_bias"] = torch.cat([sd[m + "ra.b"], sd[m + "ri.b"]], 1)
        out[a + "lam"] = sd[m + "lam"]
    elif mx.kind == "ssd":
        out[a + "in_proj.weight"] = sd[m + "in"]
        out[a + "conv_weight"], out[a + "conv_bias"] = sd[m + "conv"], sd[m + "conv.b"]
        for n in ("dt_bias", "A_log", "D"):
            out[a + n] = sd[m + n]
        out[a + "norm_weight"] = sd[m + "norm"]
    else:
        raise ValueError(f"no tensor map for mixer kind {mx.kind!r}")
    out[a + "o_proj.weight"] = sd[m + "o"]


def convert_pogorax_state_dict(sd: Dict[str, torch.Tensor], cfg: ModelConfig) -> Dict[str, torch.Tensor]:
    """Checkpoint names -> backbone parameter names."""
    out = {"model.embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"], "model.norm.weight": sd["final.norm"]}
    for i, spec in enumerate(cfg.layer_specs):
        src, dst = f"l{i}.", f"model.layers.{i}."
        out[dst + "input_layernorm.weight"] = sd[src + "norm1"]
        if spec.ff is not None:
            out[dst + "post_attention_layernorm.weight"] = sd[src + "norm2"]
            out[dst + "mlp.gate_up_proj.weight"] = torch.cat([sd[src + "mlp.gate"], sd[src + "mlp.up"]], 0)
            out[dst + "mlp.down_proj.weight"] = sd[src + "mlp.down"]
        m, a, mx = src + "mix.", dst + "self_attn.", spec.mixer
        if mx.kind == "pair":
            for j, (side, part) in enumerate(zip(("left.", "right."), mx.parts)):
                _convert_mixer(sd, m + side, f"{a}parts.{j}.", part, out)
                out[f"{a}out_norm_weights.{j}"] = sd[m + side + "out"]
        else:
            _convert_mixer(sd, m, a, mx, out)
    return out


def load_pogorax(path: str, hf_cfg: dict, dtype: torch.dtype, device: str = "cpu") -> PogoraxForCausalLM:
    from safetensors.torch import load_file

    st = os.path.join(path, "model.safetensors")
    cfg = pogorax_config(hf_cfg, read_safetensors_shapes(st))
    model = PogoraxForCausalLM(cfg)
    sd = convert_pogorax_state_dict(load_file(st), cfg)
    missing, unexpected = model.load_state_dict({k: v.to(torch.float32) for k, v in sd.items()}, strict=False)
    if missing or unexpected:
        raise RuntimeError(f"pogorax checkpoint does not fit the model: missing={missing[:6]} unexpected={unexpected[:6]}")
    model._pretrained_path = path
    return model.to(dtype).to(device)
