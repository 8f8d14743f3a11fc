"""Domorax: a decoder whose layers, in any order given by its `config.json`, mix tokens by

  * latent attention - queries through a normalised latent, keys / values rebuilt from one cached normalised latent per
    token plus one rotated key part shared by the heads (rotary frequencies stretched for long contexts), a sliding window
    and a learned sink score per head in the softmax's denominator;
  * attention whose q and k pass a short causal convolution and an RMS norm per head, whose values are the convolved keys
    before that norm, and whose scores lose a per-head slope times the distance (no other positions);
  * a gated delta rule with one decay per head behind short causal convolutions.

Every sublayer reads the fp32 residual stream itself; its OUTPUT is RMS-normalised in equal groups of channels, scaled
and added.  What a layer hands on is a learned weighted sum of the embedding output and of all layer results so far.
Dense feed-forwards use a learned mix of the first three powers of their hidden vector, each brought to unit RMS; routed
ones pick the experts of largest logit, weight them by the softmax over those logits, and add a shared expert behind a
sigmoid gate.

The model is the generic backbone (`transformer.py`) configured by `ModelConfig.layer_specs`; this module only reads the
family's `config.json` / tensor names.  A checkpoint is `config.json` + `model.safetensors` with

    embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.dwa, l<i>.mix.<name>,
    l<i>.mlp.{up, down, act} or l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down,sg}}
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from .config import ExpertFFSpec, LayerSpec, MixerSpec, ModelConfig
from .gopunex import read_safetensors_shapes
from .transformer import TransformerLMHeadModel

__all__ = ["DomoraxForCausalLM", "domorax_config", "convert_domorax_state_dict", "load_domorax"]


class DomoraxForCausalLM(TransformerLMHeadModel):
    pass


def domorax_config(hf: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> ModelConfig:
    """`shapes` (tensor name -> shape, from the checkpoint's header) settles what the config leaves to the tensors: whether
    a latent-attention layer has sink scores."""
    specs = []
    for i, ly in enumerate(hf["layers"]):
        m, kind = ly["mixer"], ly["type"]
        pre = f"l{i}.mix."
        if kind == "latent_attention":
            rot = m.get("rot") or {}
            sc = rot.get("scaling")
            mixer = MixerSpec(kind="latent", heads=m["heads"], kv_heads=1, dim=m["dim"], vdim=m["vdim"],
                              kv_rank=m["kv_rank"], rot_dim=m["rot_dim"], rot_dims=rot.get("dims", m["rot_dim"]),
                              rot_base=float(rot.get("base", 10000.0)), scale=m.get("scale"), q_rank=m.get("q_rank", 0),
                              window=(m.get("mask") or {}).get("size", 0),
                              sink_learned=shapes is None or (pre + "sink") in shapes, wide_weights=True,
                              rot_scaling=None if not sc else [float(sc["factor"]), float(sc["original"]),
                                                               float(sc["fast"]), float(sc["slow"])])
        elif kind == "attention":
            mixer = MixerSpec(kind="attention", heads=m["heads"], kv_heads=m.get("kv_heads", m["heads"]), dim=m["dim"],
                              vdim=m.get("vdim", m["dim"]), scale=m.get("scale"), conv=m.get("conv", 0), head_norm=True,
                              values_from_keys=True, dist_slopes=True, wide_weights=True)
        elif kind == "delta":
            mixer = MixerSpec(kind="delta", heads=m["heads"], kv_heads=m.get("kv_heads", m["heads"]), dim=m["dim"],
                              vdim=m.get("vdim", m["dim"]), conv=m.get("conv", 1))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = ly.get("mlp")
        if mlp is None:
            specs.append(LayerSpec(mixer=mixer))
        elif mlp.get("kind", "dense") == "dense":
            specs.append(LayerSpec(mixer=mixer, ff=mlp["ff"], ff_act="polynorm"))
        elif mlp["kind"] == "moe":
            sh = mlp.get("shared") or {}
            specs.append(LayerSpec(mixer=mixer, moe=ExpertFFSpec(
                experts=mlp["router"]["experts"], top=mlp["router"]["top"], ff=mlp["expert"]["ff"], act="silu",
                shared_ff=sh.get("ff", 0), shared_gate=bool(sh))))
        else:
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
    ffs = [s.ff for s in specs if s.ff is not None]
    return ModelConfig(model_type="domorax", vocab_size=hf["vocab"], hidden_size=hf["width"],
                       intermediate_size=max(ffs) if ffs else hf["width"], layer_specs=specs,
                       norm_eps=hf["norm"]["eps"], norm_groups=hf["norm"].get("groups", 1), norm_type="rms",
                       hidden_act="polynorm", glu=False, pos_type="none", norm_placement="sublayer_out",
                       residual_mult=hf.get("residual_mult", 1.0), fp32_residual=True, depth_average=True,
                       fp32_logits=True, tie_word_embeddings=False, max_position_embeddings=1 << 20)


def _gated(sd: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return torch.cat([sd[prefix + "gate"], sd[prefix + "up"]], 0)


def convert_domorax_state_dict(sd: Dict[str, torch.Tensor], cfg: ModelConfig) -> Dict[str, torch.Tensor]:
    """Checkpoint names -> backbone parameter names; projections that read the same input are stacked into one GEMM
    (`dq|dkv`, `q|k`, `q|k|v|b|a|g`, router + the shared expert's gate row), a layer's experts into batched tensors, the
    per-head up-projections of latent attention into [heads, ., rank]."""
    out = {"model.embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"], "model.norm.weight": sd["final.norm"]}
    for i, spec in enumerate(cfg.layer_specs):
        src, dst = f"l{i}.", f"model.layers.{i}."
        out[dst + "input_layernorm.weight"] = sd[src + "norm1"]
        out[dst + "depth_weight"] = sd[src + "dwa"]
        if spec.ff is not None or spec.moe is not None:
            out[dst + "post_attention_layernorm.weight"] = sd[src + "norm2"]
        if spec.ff is not None:
            out[dst + "mlp.up_proj.weight"] = sd[src + "mlp.up"]
            out[dst + "mlp.down_proj.weight"] = sd[src + "mlp.down"]
            out[dst + "mlp.act_coef"] = sd[src + "mlp.act"]
        elif spec.moe is not None:
            p = src + "mlp."
            out[dst + "mlp.router.weight"] = torch.cat([sd[p + "router"], sd[p + "shared.sg"]], 0) if spec.moe.shared_gate \
                else sd[p + "router"]
            out[dst + "mlp.experts.w_up"] = torch.stack([_gated(sd, f"{p}e{e}.") for e in range(spec.moe.experts)])
            out[dst + "mlp.experts.w_down"] = torch.stack([sd[f"{p}e{e}.down"] for e in range(spec.moe.experts)])
            if spec.moe.shared_ff:
                out[dst + "mlp.shared.gate_up_proj.weight"] = _gated(sd, p + "shared.")
                out[dst + "mlp.shared.down_proj.weight"] = sd[p + "shared.down"]
        m, a, mx = src + "mix.", dst + "self_attn.", spec.mixer
        if mx.kind == "latent":
            if mx.q_rank:
                out[a + "in_proj.weight"] = torch.cat([sd[m + "dq"], sd[m + "dkv"]], 0)
                out[a + "dq_norm_weight"] = sd[m + "dq.norm"]
                out[a + "uq_proj.weight"] = sd[m + "uq"]
            else:
                out[a + "in_proj.weight"] = torch.cat([sd[m + "q"], sd[m + "dkv"]], 0)
            out[a + "dkv_norm_weight"] = sd[m + "dkv.norm"]
            out[a + "uk"] = sd[m + "uk"].reshape(mx.heads, mx.dim, mx.kv_rank)
            out[a + "uv"] = sd[m + "uv"].reshape(mx.heads, mx.vdim, mx.kv_rank)
            if mx.sink_learned:
                out[a + "sink_logit"] = sd[m + "sink"]
        elif mx.kind == "attention":
            out[a + "qkv_proj.weight"] = torch.cat([sd[m + "q"], sd[m + "k"]], 0)
            if mx.conv:
                out[a + "conv_weight"] = torch.cat([sd[m + "q.conv"], sd[m + "k.conv"]], 0)
            out[a + "q_head_norm_weight"] = sd[m + "q.norm"]
            out[a + "k_head_norm_weight"] = sd[m + "k.norm"]
        else:
            out[a + "in_proj.weight"] = torch.cat([sd[m + "q"], sd[m + "k"], sd[m + "v"], sd[m + "b"], sd[m + "a"],
                                                   sd[m + "g"]], 0)
            out[a + "conv_weight"] = torch.cat([sd[m + "q.conv"], sd[m + "k.conv"], sd[m + "v.conv"]], 0)
            out[a + "A_log"] = sd[m + "A_log"]
            out[a + "dt_bias"] = sd[m + "dt_bias"]
            out[a + "norm_weight"] = sd[m + "norm"]
        out[a + "o_proj.weight"] = sd[m + "o"]
    return out


def load_domorax(path: str, hf_cfg: dict, dtype: torch.dtype, device: str = "cpu") -> DomoraxForCausalLM:
    from safetensors.torch import load_file

    st = os.path.join(path, "model.safetensors")
    cfg = domorax_config(hf_cfg, read_safetensors_shapes(st))
    model = DomoraxForCausalLM(cfg)
    sd = convert_domorax_state_dict(load_file(st), cfg)
    missing, unexpected = model.load_state_dict({k: v.to(torch.float32) for k, v in sd.items()}, strict=False)
    if missing or unexpected:
        raise RuntimeError(f"domorax checkpoint does not fit the model: missing={missing[:6]} unexpected={unexpected[:6]}")
    model._pretrained_path = path
    return model.to(dtype).to(device)
