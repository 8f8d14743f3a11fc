"""Typed model configs + the zoo of named presets used by examples, tests and bench.py.

Parity: the model table in reference `examples/language/llama/benchmark.py:33-59` (100m/5b/7b/13b/70b) plus the
HF config fields the reference's policies read (`shardformer/policies/*.py`).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Any, Dict, List, Optional, Tuple

__all__ = ["ModelConfig", "MoEConfig", "MixerSpec", "ExpertFFSpec", "LayerSpec", "MODEL_ZOO", "get_config"]


@dataclass
class MoEConfig:
    num_experts: int = 8
    top_k: int = 2
    moe_intermediate_size: Optional[int] = None  # per-expert FFN width (defaults to intermediate_size)
    n_shared_experts: int = 0                     # DeepSeekMoE shared experts
    first_k_dense_replace: int = 0                # leading dense layers (DeepSeek)
    moe_layer_freq: int = 1
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.02
    router_z_loss_coef: float = 0.0
    scoring_func: str = "softmax"                 # "softmax" | "sigmoid" (DeepSeek-V3)
    n_group: int = 1                              # grouped top-k (DeepSeek-V3)
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    capacity_factor: float = 0.0                  # 0 = dropless


@dataclass
class MixerSpec:
    """The token mixer of one layer of a hybrid decoder (`ModelConfig.layer_specs`).

    kind "attention":  softmax attention over a paged cache; q/k heads `dim` wide, value heads `vdim` wide; optional
                       learned bias per (distance bucket, head) with `bias_buckets` rows (first half exact distances,
                       second half logarithmic up to `bias_max`), optional zero-score `sink` in the softmax denominator,
                       optional RMS norm over the whole q / k projection, optional blend of the values with those of the
                       first `v_mix` layer.
    kind "lightning":  per-head outer-product memory with one scalar `decay` per head, read out by q.
    kind "channel_delta": gated delta rule with a decay per head and key channel, short causal convolutions of `conv`
                       taps on q, k, v, low-rank (`decay_rank`, `gate_rank`) projections for the decay and output gate.
    kind "latent":     softmax attention whose keys and values are rebuilt from one `kv_rank`-wide normalised latent per
                       token plus one `rot_dim`-wide rotated key part shared by all heads; q heads are `dim` unrotated +
                       `rot_dim` rotated channels; only the latent and the rotated part are cached.
    kind "retention":  outer-product memory per head with one scalar `decay` per head, rotary positions on the first
                       `rot_dims` channels of q and k (base `rot_base`), k scaled by dim^-1/2, no softmax; the read-out
                       is brought to unit RMS per head and gated.
    kind "mlstm":      matrix memory with exponential gating: per head a log input gate and a log forget gate (both
                       soft-capped at `gate_cap`), a running maximum that keeps the exponentials bounded, a normaliser
                       vector beside the matrix; the read-out is divided by max(|n . q|, exp(-m)), brought to unit RMS
                       per head, weighted and gated by a sigmoid.
    kind "ssd":        selective state space (state-space duality form): `heads` x `vdim` inner channels, `state` rows per
                       head, B / C shared by `groups` of heads, a causal convolution of `conv` taps (with bias) and silu
                       on x | B | C, step size softplus(dt + bias), decay exp(-exp(A_log) dt), skip D x, the output gated by
                       silu(z) BEFORE an RMS norm in `norm_groups` parts.
    kind "rglru":      gated linear recurrent unit per channel (`lru_width` channels, gates from block-diagonal matrices of
                       `blocks` blocks, decay exp(-`lru_c` r softplus(lam))) behind a causal convolution of `conv` taps,
                       multiplied by a tanh-GELU branch.
    kind "pair":       several mixers side by side that read the same input (`parts`); every part's output is RMS-normed
                       over the model width with a weight of its own and the results are averaged.
    kind "delta":      gated delta rule with ONE decay per head, exp(-exp(A_log) softplus(W_a h + dt_bias)), a write
                       strength sigmoid(W_b h), short causal convolutions of `conv` taps + silu on q, k, v, unit-length
                       q / k, the read-out brought to unit RMS per head, weighted and gated by silu(W_g h).

    kind "latent" also takes: `q_rank` (queries through an RMS-normalised latent of that width), `window`,
    `sink_learned`, `rot_scaling`.

    kind "attention" also takes: rotary positions on the first `rot_dims` channels of every q / k head (pairs (2i, 2i + 1)
    when `rot_interleaved`, else (i, i + rot_dims / 2)); `head_unit_norm` (q and k divided by their root mean square over
    the head, after the rotation, no weight); `mask_block` (a position sees only the keys of its own block of that many
    positions, counted from the start of the sequence); `out_gate` (heads times sigmoid(W_g x) before the output
    projection); `conv` (a causal convolution of that many taps on every channel of the q and k projections, no
    activation; its last inputs are carried like a recurrent state); `head_norm` (RMS norm of every q / k head with one
    weight over the head's channels per projection); `values_from_keys` (no value projection: the values are the keys as
    they leave the convolution, before any norm); `dist_slopes` (score minus 2^(-8 (h + 1) / heads) x distance);
    `window` (a position sees itself and the window - 1 positions before it); `sink_learned` (the sink's score is a
    learned number per head instead of 0)."""

    kind: str = "attention"
    heads: int = 1
    kv_heads: Optional[int] = None
    dim: int = 64
    vdim: Optional[int] = None
    bias: bool = False
    scale: Optional[float] = None
    bias_buckets: int = 0
    bias_max: float = 0.0
    sink: bool = False
    proj_norm: bool = False
    v_mix: bool = False
    decay: Optional[List[float]] = None
    conv: int = 0
    decay_rank: int = 0
    gate_rank: int = 0
    kv_rank: int = 0
    rot_dim: int = 0                  # width of the decoupled rotated q / k part (latent attention)
    rot_dims: int = 0                 # channels of a head that rotary positions turn (rotate-half pairs)
    rot_base: float = 10000.0
    rot_interleaved: bool = False     # rotary pairs are (2i, 2i + 1) instead of (i, i + rot_dims / 2)
    head_unit_norm: bool = False      # q, k / rms over the head (after the rotation), no weight
    mask_block: int = 0               # > 0: keys of the query's own block of this many positions only
    out_gate: bool = False            # heads * sigmoid(W_g x) in front of the output projection
    wide_weights: bool = False        # 16-bit serving: softmax weights enter the weighted sum with ~16 bits of mantissa
    gate_cap: float = 0.0             # mlstm: soft cap of the gate pre-activations (0 = none)
    state: int = 0                    # ssd: rows of a head's state
    groups: int = 1                   # ssd: groups of heads that share B / C
    norm_groups: int = 1              # ssd: parts of the gated RMS norm
    lru_width: int = 0                # rglru: channels
    blocks: int = 1                   # rglru: blocks of the gate matrices
    lru_c: float = 8.0                # rglru: decay = exp(-lru_c * r * softplus(lam))
    q_rank: int = 0                   # latent: width of the normalised query latent (0 = queries straight from the input)
    window: int = 0                   # attention / latent: > 0 keeps the keys pos - window + 1 .. pos
    sink_learned: bool = False        # the softmax sink's score is a learned number per head (implies a sink)
    rot_scaling: Optional[List[float]] = None     # (factor, original length, fast, slow): stretched slow frequencies
    head_norm: bool = False           # attention: RMS norm per q / k head with a weight shared by the heads
    values_from_keys: bool = False    # attention: values = keys before their norm (no value projection)
    dist_slopes: bool = False         # attention: score -= 2^(-8 (h + 1) / heads) * (query position - key position)
    parts: Optional[List["MixerSpec"]] = None      # pair: the mixers that run side by side

    def __post_init__(self) -> None:
        if self.kv_heads is None:
            self.kv_heads = self.heads
        if self.vdim is None:
            self.vdim = self.dim
        assert self.heads % self.kv_heads == 0, "query heads must be a multiple of key/value heads"
        if self.parts is not None:
            self.parts = [MixerSpec(**p) if isinstance(p, dict) else p for p in self.parts]
            assert sum(p.paged for p in self.parts) <= 1 and sum(p.recurrent for p in self.parts) <= 1, \
                "a pair holds at most one paged and one recurrent mixer (they share the layer's pages / state slot)"

    @property
    def recurrent(self) -> bool:
        if self.kind == "pair":
            return any(p.recurrent for p in self.parts)
        if self.kind == "attention":                  # a convolution in front of attention carries its last inputs
            return self.conv > 0
        return self.kind in ("lightning", "channel_delta", "retention", "mlstm", "ssd", "rglru", "delta")

    @property
    def paged(self) -> bool:
        if self.kind == "pair":
            return any(p.paged for p in self.parts)
        return self.kind in ("attention", "latent")

    @property
    def paged_part(self) -> Optional["MixerSpec"]:
        """The mixer that owns the layer's pages (itself, or the paged part of a pair)."""
        if self.kind == "pair":
            return next((p for p in self.parts if p.paged), None)
        return self if self.paged else None

    @property
    def recurrent_part(self) -> Optional["MixerSpec"]:
        if self.kind == "pair":
            return next((p for p in self.parts if p.recurrent), None)
        return self if self.recurrent else None


@dataclass
class ExpertFFSpec:
    """Routed feed-forward of one layer: `experts` gated experts of width `ff`, every token uses the `top` of largest
    softmax score (weights renormalised to one), plus an optional shared expert of width `shared_ff` for every token.
    Expert activation `act`: "clamped": g = min(gate, limit), u = clamp(up, -limit, limit),
    y = g * sigmoid(alpha * g) * (u + 1); "silu": y = silu(gate) * up.  `shared_gate`: the shared expert's output is
    multiplied by sigmoid(w_sg . h), one number per token.  (Softmax over all experts renormalised over the chosen ones
    equals the softmax over the chosen logits alone.)"""

    experts: int = 1
    top: int = 1
    ff: int = 0
    limit: float = 7.0
    alpha: float = 1.702
    shared_ff: int = 0
    shared_limit: float = 7.0
    act: str = "clamped"
    shared_gate: bool = False


@dataclass
class LayerSpec:
    mixer: MixerSpec = field(default_factory=MixerSpec)
    ff: Optional[int] = None          # dense feed-forward width; None = no dense feed-forward
    moe: Optional[ExpertFFSpec] = None  # routed feed-forward instead of a dense one
    ff_act: Optional[str] = None      # dense feed-forward: activation of this layer instead of `ModelConfig.hidden_act`
                                      # ("polynorm": learned mix of the first three powers, each brought to unit RMS)

    def __post_init__(self) -> None:
        if isinstance(self.mixer, dict):
            self.mixer = MixerSpec(**self.mixer)
        if isinstance(self.moe, dict):
            self.moe = ExpertFFSpec(**self.moe)


@dataclass
class ModelConfig:
    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    max_position_embeddings: int = 4096
    norm_eps: float = 1e-5
    norm_type: str = "rms"            # "rms" | "layer"
    hidden_act: str = "silu"
    glu: bool = True                  # gated MLP (SwiGLU / GeGLU) vs. plain 2-layer MLP
    attention_bias: bool = False
    attention_out_bias: Optional[bool] = None
    mlp_bias: bool = False
    pos_type: str = "rope"            # "rope" | "learned" | "alibi" | "none"
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    rope_interleaved: bool = False    # GPT-J / ChatGLM pair layout
    partial_rotary_factor: float = 1.0
    qk_norm: bool = False             # Qwen3 / Cohere per-head q/k norm
    parallel_block: bool = False      # attn and mlp read the same normed input (GPT-J, Falcon, Cohere)
    tie_word_embeddings: bool = False
    causal: bool = True
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    type_vocab_size: int = 0          # BERT token types
    post_norm: bool = False           # BERT-style post-LN
    final_norm: bool = True
    embed_norm: bool = False          # Bloom / BERT embedding layernorm
    initializer_range: float = 0.02
    attn_dropout: float = 0.0
    hidden_dropout: float = 0.0
    sliding_window: Optional[int] = None
    lm_head_bias: bool = False        # GPT-J
    norm_head: bool = False           # Baichuan-2 NormHead: L2-normalised LM-head rows
    moe: Optional[MoEConfig] = None
    # multi-head latent attention (DeepSeek-V2 / V3): low-rank q and kv projections, decoupled rope key
    q_lora_rank: Optional[int] = None
    kv_lora_rank: Optional[int] = None
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # hybrid decoders: one spec per layer (mixer kind and sizes, feed-forward width) instead of the uniform fields above
    layer_specs: Optional[List[LayerSpec]] = None
    norm_placement: str = "pre"       # "pre": sublayer(norm(x)); "sublayer_out": x + residual_mult * norm(sublayer(x))
    residual_mult: float = 1.0
    norm_weight_offset: float = 0.0   # zero-centred norm weights: the norm multiplies by (offset + w)
    fp32_residual: bool = False       # the residual stream stays in fp32 whatever the compute dtype
    norm_bias: bool = True            # layer norms carry a bias
    logit_softcap: Optional[float] = None   # logits <- cap * tanh(logits / cap), after `logit_scale`
    fp32_logits: bool = False         # 16-bit serving keeps the LM head's fp32 accumulator (no 16-bit rounding of logits)
    norm_groups: int = 1              # "sublayer_out" norms and the final norm: RMS over each of this many equal parts
    depth_average: bool = False       # what a layer hands on is a learned weighted sum of the embedding output and of
                                      # all layer results so far (one weight vector per layer)
    # looped span: layers loop_start .. loop_stop-1 run `loop_times` times in a row with the same weights; every pass
    # has caches / states of its own and starts by adding the embedding output (not the first pass) and a learned
    # vector of the pass to the stream
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    pad_token_id: Optional[int] = None
    bos_token_id: int = 1
    eos_token_id: int = 2

    def __post_init__(self) -> None:
        if self.layer_specs is not None:
            self.layer_specs = [LayerSpec(**s) if isinstance(s, dict) else s for s in self.layer_specs]
            self.num_hidden_layers = len(self.layer_specs)
            att = [s.mixer.paged_part for s in self.layer_specs if s.mixer.paged] or [self.layer_specs[0].mixer]
            self.num_attention_heads, self.num_key_value_heads, self.head_dim = att[0].heads, att[0].kv_heads, att[0].dim
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.kv_lora_rank is not None:
            # MLA: q / k heads are nope + rope wide (the KV cache stores that width; v is padded up to it)
            self.head_dim = self.qk_nope_head_dim + self.qk_rope_head_dim
            self.num_key_value_heads = self.num_attention_heads
            self.v_head_dim = self.v_head_dim or self.head_dim
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.attention_out_bias is None:
            self.attention_out_bias = self.attention_bias
        if isinstance(self.moe, dict):
            self.moe = MoEConfig(**self.moe)

    @property
    def looped(self) -> bool:
        return self.loop_stop > self.loop_start

    def layer_runs(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, pass) in execution order; pass is None outside the looped span.  The index into this list is the
        layer run's cache index: a layer of the span owns one cache / state per pass."""
        n = self.num_hidden_layers
        if not self.looped:
            return [(i, None) for i in range(n)]
        a, b = self.loop_start, self.loop_stop
        return [(i, None) for i in range(a)] + [(i, t) for t in range(self.loop_times) for i in range(a, b)] + \
            [(i, None) for i in range(b, n)]

    @property
    def num_cache_layers(self) -> int:
        return len(self.layer_runs())

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def use_mla(self) -> bool:
        return self.kv_lora_rank is not None

    @property
    def rotary_dim(self) -> int:
        if self.use_mla:
            return self.qk_rope_head_dim
        return int(self.head_dim * self.partial_rotary_factor)

    def num_params(self, include_embeddings: bool = True) -> int:
        h, L = self.hidden_size, self.num_hidden_layers
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.moe is not None:
            ei = self.moe.moe_intermediate_size or self.intermediate_size
            per_expert = h * ei * (3 if self.glu else 2)
            mlp = per_expert * (self.moe.num_experts + self.moe.n_shared_experts) + h * self.moe.num_experts
        else:
            mlp = h * self.intermediate_size * (3 if self.glu else 2)
        n = L * (attn + mlp + 2 * h) + h
        if include_embeddings:
            n += self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return n

    def flops_per_token(self, seq_len: int, backward: bool = True, checkpoint: bool = False) -> float:
        """Model FLOPs per token (matmul only; causal attention counted at half)."""
        h, L = self.hidden_size, self.num_hidden_layers
        attn_proj = 2 * h * (self.q_size + 2 * self.kv_size) + 2 * self.q_size * h
        if self.moe is not None:
            ei = self.moe.moe_intermediate_size or self.intermediate_size
            act = self.moe.top_k + self.moe.n_shared_experts
            mlp = 2 * h * ei * (3 if self.glu else 2) * act
        else:
            mlp = 2 * h * self.intermediate_size * (3 if self.glu else 2)
        attn_sdp = 4 * seq_len * self.q_size * (0.5 if self.causal else 1.0)
        fwd = L * (attn_proj + mlp + attn_sdp) + 2 * h * self.vocab_size
        mult = (3.0 if backward else 1.0) + (1.0 if (checkpoint and backward) else 0.0)
        return fwd * mult

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def replace(self, **kw) -> "ModelConfig":
        return replace(self, **kw)


def _llama(**kw) -> ModelConfig:
    return ModelConfig(model_type="llama", **kw)


MODEL_ZOO: Dict[str, ModelConfig] = {
    # ---- reference benchmark table (Llama-2 shapes, examples/language/llama/benchmark.py:33-59)
    "llama-100m": _llama(hidden_size=1024, intermediate_size=2048, num_hidden_layers=4, num_attention_heads=32),
    "llama-5b": _llama(num_key_value_heads=8),
    "llama2-7b": _llama(),
    "llama2-13b": _llama(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40),
    "llama2-70b": _llama(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                         num_key_value_heads=8),
    # ---- Llama-3 (BASELINE.json flagship)
    "llama3-8b": _llama(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                        num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=8192,
                        rope_theta=500000.0),
    "llama3-70b": _llama(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                         num_attention_heads=64, num_key_value_heads=8, max_position_embeddings=8192,
                         rope_theta=500000.0),
    "llama-tiny": _llama(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256),
    # ---- MoE
    "mixtral-8x7b": ModelConfig(model_type="mixtral", vocab_size=32000, hidden_size=4096, intermediate_size=14336,
                                num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                                max_position_embeddings=32768, rope_theta=1e6,
                                moe=MoEConfig(num_experts=8, top_k=2)),
    "mixtral-tiny": ModelConfig(model_type="mixtral", vocab_size=512, hidden_size=64, intermediate_size=128,
                                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                max_position_embeddings=256, moe=MoEConfig(num_experts=4, top_k=2)),
    "deepseek-moe-16b": ModelConfig(model_type="deepseek", vocab_size=102400, hidden_size=2048,
                                    intermediate_size=10944, num_hidden_layers=28, num_attention_heads=16,
                                    max_position_embeddings=4096,
                                    moe=MoEConfig(num_experts=64, top_k=6, moe_intermediate_size=1408,
                                                  n_shared_experts=2, first_k_dense_replace=1, norm_topk_prob=False)),
    "deepseek-tiny": ModelConfig(model_type="deepseek", vocab_size=512, hidden_size=64, intermediate_size=128,
                                 num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=256,
                                 moe=MoEConfig(num_experts=8, top_k=2, moe_intermediate_size=32, n_shared_experts=1,
                                               first_k_dense_replace=1, norm_topk_prob=False)),
    # ---- DeepSeek-V3: MLA + sigmoid router with group-limited top-k, shared expert, first 3 layers dense
    "deepseek-v3": ModelConfig(model_type="deepseek_v3", vocab_size=129280, hidden_size=7168, intermediate_size=18432,
                               num_hidden_layers=61, num_attention_heads=128, max_position_embeddings=163840,
                               norm_eps=1e-6, rope_theta=10000.0, rope_interleaved=True, q_lora_rank=1536,
                               kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                               moe=MoEConfig(num_experts=256, top_k=8, moe_intermediate_size=2048, n_shared_experts=1,
                                             first_k_dense_replace=3, norm_topk_prob=True, scoring_func="sigmoid",
                                             n_group=8, topk_group=4, routed_scaling_factor=2.5)),
    "deepseek_v3-tiny": ModelConfig(model_type="deepseek_v3", vocab_size=512, hidden_size=64, intermediate_size=128,
                                    num_hidden_layers=3, num_attention_heads=4, max_position_embeddings=256,
                                    norm_eps=1e-6, rope_interleaved=True, q_lora_rank=24, kv_lora_rank=16,
                                    qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=12,
                                    moe=MoEConfig(num_experts=8, top_k=2, moe_intermediate_size=32, n_shared_experts=1,
                                                  first_k_dense_replace=1, norm_topk_prob=True, scoring_func="sigmoid",
                                                  n_group=4, topk_group=2, routed_scaling_factor=2.5)),
    # ---- GPT-2 family (learned positions, LayerNorm, GELU, tied embeddings)
    "gpt2": ModelConfig(model_type="gpt2", vocab_size=50257, hidden_size=768, intermediate_size=3072,
                        num_hidden_layers=12, num_attention_heads=12, max_position_embeddings=1024, norm_type="layer",
                        hidden_act="gelu_new", glu=False, attention_bias=True, mlp_bias=True, pos_type="learned",
                        tie_word_embeddings=True),
    "gpt2-tiny": ModelConfig(model_type="gpt2", vocab_size=512, hidden_size=64, intermediate_size=256,
                             num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=128,
                             norm_type="layer", hidden_act="gelu_new", glu=False, attention_bias=True, mlp_bias=True,
                             pos_type="learned", tie_word_embeddings=True),
    "mistral-7b": ModelConfig(model_type="mistral", vocab_size=32000, hidden_size=4096, intermediate_size=14336,
                              num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                              max_position_embeddings=32768, sliding_window=4096),
    "qwen2-7b": ModelConfig(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                            num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
                            max_position_embeddings=32768, rope_theta=1e6, attention_bias=True,
                            attention_out_bias=False, norm_eps=1e-6),
    "qwen3-8b": ModelConfig(model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                            num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                            max_position_embeddings=40960, rope_theta=1e6, qk_norm=True, norm_eps=1e-6),
    "bert-base": ModelConfig(model_type="bert", vocab_size=30522, hidden_size=768, intermediate_size=3072,
                             num_hidden_layers=12, num_attention_heads=12, max_position_embeddings=512,
                             norm_type="layer", hidden_act="gelu", glu=False, attention_bias=True, mlp_bias=True,
                             pos_type="learned", causal=False, type_vocab_size=2, post_norm=True, final_norm=False,
                             embed_norm=True, norm_eps=1e-12),
    "opt-125m": ModelConfig(model_type="opt", vocab_size=50272, hidden_size=768, intermediate_size=3072,
                            num_hidden_layers=12, num_attention_heads=12, max_position_embeddings=2048,
                            norm_type="layer", hidden_act="relu", glu=False, attention_bias=True, mlp_bias=True,
                            pos_type="learned", tie_word_embeddings=True),
    "bloom-560m": ModelConfig(model_type="bloom", vocab_size=250880, hidden_size=1024, intermediate_size=4096,
                              num_hidden_layers=24, num_attention_heads=16, norm_type="layer", hidden_act="gelu_new",
                              glu=False, attention_bias=True, mlp_bias=True, pos_type="alibi", embed_norm=True,
                              tie_word_embeddings=True),
    "falcon-7b": ModelConfig(model_type="falcon", vocab_size=65024, hidden_size=4544, intermediate_size=18176,
                             num_hidden_layers=32, num_attention_heads=71, num_key_value_heads=1, norm_type="layer",
                             hidden_act="gelu", glu=False, parallel_block=True),
    "gptj-6b": ModelConfig(model_type="gptj", vocab_size=50400, hidden_size=4096, intermediate_size=16384,
                           num_hidden_layers=28, num_attention_heads=16, max_position_embeddings=2048,
                           norm_type="layer", hidden_act="gelu_new", glu=False, mlp_bias=True, parallel_block=True,
                           rope_interleaved=True, partial_rotary_factor=0.25, lm_head_bias=True),
    "chatglm2-6b": ModelConfig(model_type="chatglm", vocab_size=65024, hidden_size=4096, intermediate_size=13696,
                               num_hidden_layers=28, num_attention_heads=32, num_key_value_heads=2,
                               max_position_embeddings=32768, attention_bias=True, attention_out_bias=False,
                               rope_interleaved=True, partial_rotary_factor=0.5),
    "baichuan-7b": ModelConfig(model_type="baichuan", vocab_size=64000, hidden_size=4096, intermediate_size=11008,
                               num_hidden_layers=32, num_attention_heads=32, max_position_embeddings=4096,
                               norm_eps=1e-6),
    "baichuan2-13b": ModelConfig(model_type="baichuan", vocab_size=125696, hidden_size=5120, intermediate_size=13696,
                                 num_hidden_layers=40, num_attention_heads=40, max_position_embeddings=4096,
                                 pos_type="alibi", norm_eps=1e-6, norm_head=True),
    "baichuan-tiny": ModelConfig(model_type="baichuan", vocab_size=512, hidden_size=64, intermediate_size=128,
                                 num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=256,
                                 pos_type="alibi", norm_head=True),
    "command-r": ModelConfig(model_type="command", vocab_size=256000, hidden_size=8192, intermediate_size=22528,
                             num_hidden_layers=40, num_attention_heads=64, num_key_value_heads=64, norm_type="layer",
                             parallel_block=True, tie_word_embeddings=True, logit_scale=0.0625, rope_theta=8e6,
                             rope_interleaved=True),
}


def _tiny(preset: str, **kw) -> ModelConfig:
    """Test-size variant of a family preset (2 layers, hidden 64, 4 heads, vocab 512) keeping every family switch."""
    base = dict(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=None, max_position_embeddings=256)
    base.update(kw)
    return replace(MODEL_ZOO[preset], **base)


MODEL_ZOO.update({
    "mistral-tiny": _tiny("mistral-7b", sliding_window=None),
    "qwen2-tiny": _tiny("qwen2-7b"),
    "qwen3-tiny": _tiny("qwen3-8b", head_dim=16),
    "opt-tiny": _tiny("opt-125m", num_key_value_heads=4),
    "bloom-tiny": _tiny("bloom-560m", num_key_value_heads=4),
    "falcon-tiny": _tiny("falcon-7b", num_key_value_heads=2),
    "gptj-tiny": _tiny("gptj-6b", num_key_value_heads=4, partial_rotary_factor=0.5),
    "chatglm-tiny": _tiny("chatglm2-6b"),
    "command-tiny": _tiny("command-r", num_key_value_heads=4),
    "bert-tiny": _tiny("bert-base", num_key_value_heads=4),
})


def get_config(name: str, **overrides) -> ModelConfig:
    if name not in MODEL_ZOO:
        raise KeyError(f"unknown model preset {name!r}; available: {sorted(MODEL_ZOO)}")
    cfg = MODEL_ZOO[name]
    if not overrides:
        return replace(cfg)
    # derived fields must be re-derived when the shape changes
    if ("hidden_size" in overrides or "num_attention_heads" in overrides) and "head_dim" not in overrides \
            and cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads:
        overrides["head_dim"] = None
    return replace(cfg, **overrides)
