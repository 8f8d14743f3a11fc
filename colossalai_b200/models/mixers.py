"""Token mixers of hybrid decoders, beside the rotary / ALiBi `Attention` of `transformer.py`:

  * `BiasSinkAttention`: softmax attention over the paged cache with a learned bias per (distance bucket, head), a
    zero-score sink in the denominator, an RMS norm over the whole q / k projection and a blend of the values with
    those of the first value-mixing layer;
  * `LightningAttention`: linear attention with one scalar decay per head (an outer-product memory per head);
  * `ChannelDeltaMixer`: gated delta rule with a decay per head and key channel and short causal convolutions;
  * `LatentAttention`: softmax attention whose keys / values are rebuilt from one small normalised latent per token plus
    one rotated key part shared by all heads - only those are cached, and the attention runs in the latent space;
  * `Retention`: decayed outer-product memory per head with rotary positions on q / k, no softmax, unit-RMS gated read-out;
  * `MatrixLSTM`: matrix memory with exponential input / forget gates, a running maximum and a normaliser vector;
  * `SelectiveStateSpace`: state space with input-dependent step sizes behind a causal convolution, gate before the norm;
  * `GatedLinearRecurrence`: per-channel real-gated linear recurrent unit behind a causal convolution, times a GELU branch;
  * `MixerPair`: mixers side by side on the same input; their RMS-normed outputs are averaged;
  * `DeltaMixer`: gated delta rule with one decay per head behind short causal convolutions, gated unit-RMS read-out.

`BiasSinkAttention` also covers plain paged softmax attention with rotary positions (half or interleaved pairs, on a part
of the head), a weightless unit norm of q / k heads, a block mask (a position sees its own block of positions only), a
sigmoid output gate, a short convolution on q | k, an RMS norm per q / k head with a shared weight, values taken from the
keys, a linear distance penalty per head, a sliding window and a learned sink score: every one of these is a field of the
`MixerSpec`.

Every mixer keeps the call signature of `Attention` (`forward(x, meta, rope, kv_cache)`) and is selected per layer by
`ModelConfig.layer_specs[i].mixer.kind` (`build_mixer`).  `kv_cache` is the step runtime (`inference.modeling.PagedKVRuntime`):
it carries the ragged layout of the step, the paged K / V of attention layers and the per-slot recurrent state of the
others, so a whole prompt, a portion of one and a single decoded token all take the same path.  Sizes and constants come
from the `MixerSpec`; what the design fixes (activation choices, where the unit norm sits) is in the code.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import mixers as mops
from .config import MixerSpec, ModelConfig

__all__ = ["BiasSinkAttention", "LightningAttention", "ChannelDeltaMixer", "LatentAttention", "Retention", "MatrixLSTM",
           "SelectiveStateSpace", "GatedLinearRecurrence", "MixerPair", "DeltaMixer", "build_mixer"]


class _MixerBase(nn.Module):
    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__()
        self.cfg, self.spec, self.layer_idx = cfg, spec, layer_idx
        self.shard_config = None
        self._aux_cache: Dict[Tuple[str, str], torch.Tensor] = {}

    def _aux(self, name: str, device, make) -> torch.Tensor:
        """Small constant tensors in exact fp32 / int32 on the compute device (built once per device)."""
        key = (name, str(device))
        if key not in self._aux_cache:
            self._aux_cache[key] = make().to(device)
        return self._aux_cache[key]

    def _apply(self, fn, *a, **k):          # parameters moved or cast: the derived constants are rebuilt
        self._aux_cache = {}
        return super()._apply(fn, *a, **k)


class BiasSinkAttention(_MixerBase):
    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        H, G, d, dv = spec.heads, spec.kv_heads, spec.dim, spec.vdim
        assert spec.rot_dims % 2 == 0 and spec.rot_dims <= d
        assert not spec.values_from_keys or (dv == d and not spec.v_mix), "values taken from the keys are key-wide"
        assert not (spec.conv and (spec.rot_dims or spec.head_unit_norm or spec.proj_norm)), \
            "the convolution on q | k is followed by the per-head norm only"
        # q | k | v (| output gate): one GEMM reads the layer input (no v with `values_from_keys`)
        self.v_width = 0 if spec.values_from_keys else G * dv
        self.qkv_proj = nn.Linear(cfg.hidden_size, H * d + G * d + self.v_width + (H * dv if spec.out_gate else 0),
                                  bias=spec.bias)
        if spec.conv:
            self.conv_weight = nn.Parameter(torch.zeros((H + G) * d, spec.conv))       # q channels, then k channels
        if spec.head_norm:
            self.q_head_norm_weight = nn.Parameter(torch.ones(d))
            self.k_head_norm_weight = nn.Parameter(torch.ones(d))
        if spec.sink_learned:
            self.sink_logit = nn.Parameter(torch.zeros(H))
        if spec.proj_norm:
            self.q_norm_weight = nn.Parameter(torch.ones(H * d))
            self.k_norm_weight = nn.Parameter(torch.ones(G * d))
        if spec.bias_buckets:
            self.rel_bias = nn.Parameter(torch.zeros(spec.bias_buckets, H))
        if spec.v_mix:
            self.v_mix = nn.Parameter(torch.zeros(()))
        self.o_proj = nn.Linear(H * dv, cfg.hidden_size, bias=False)
        self.scale = spec.scale if spec.scale is not None else d ** -0.5

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp, eps = self.spec, self.cfg.norm_eps
        H, G, d, dv = sp.heads, sp.kv_heads, sp.dim, sp.vdim
        qkv = self.qkv_proj(x)
        q, k, v, gate = qkv.split([H * d, G * d, self.v_width, H * dv if sp.out_gate else 0], dim=-1)
        if sp.conv:
            # the convolution comes directly after the projection; its window of last inputs lives in the layer's slot
            qk = mops.short_conv_silu(qkv[:, : (H + G) * d], self.conv_weight, kv_cache.layer_state(self.layer_idx)["conv"],
                                      kv_cache.ragged, activation=False)
            q, k = qk[:, : H * d], qk[:, H * d:]
        if sp.values_from_keys:
            v = k                                          # as they leave the convolution, before the norm
        if sp.head_norm and sp.values_from_keys:
            # one pass: normed query heads out, normed key heads into the key pages, un-normed ones into the value pages
            kc, vc = kv_cache.pages(self.layer_idx)
            q = mops.head_rms_norm(qk if sp.conv else qkv, H, G, d, self.q_head_norm_weight, self.k_head_norm_weight, eps,
                                   pages=(kc, vc, kv_cache.block_tables, kv_cache.ragged))
            k = v = None
        elif sp.head_norm:
            qk = mops.head_rms_norm(qk if sp.conv else qkv, H, G, d, self.q_head_norm_weight, self.k_head_norm_weight, eps)
            q, k = qk[:, : H * d], qk[:, H * d:]
        if sp.rot_dims or sp.head_unit_norm:
            # q and k heads sit side by side in the projection: rotated and normalised in place, in one launch
            table = mops.rotary_table(kv_cache.max_len_host, sp.rot_dims, sp.rot_base, x.device) if sp.rot_dims else None
            mops.rotary_unit_norm(qkv, H + G, d, sp.rot_dims, sp.rot_interleaved, table, kv_cache.ragged.token_pos,
                                  eps if sp.head_unit_norm else None)
        if sp.proj_norm:
            q = ops.rms_norm(q.contiguous(), self.q_norm_weight, eps)
            k = ops.rms_norm(k.contiguous(), self.k_norm_weight, eps)
        v_other, lam = None, 0.0
        if sp.v_mix:
            first = kv_cache.shared.get("v_first")
            if first is None:
                kv_cache.shared["v_first"] = v          # the first value-mixing layer lends its values, unblended
            else:
                v_other = first
                lam = self._aux("lam", "cpu", lambda: self.v_mix.detach().float().cpu()).item()
        table = starts = lut = None
        if sp.bias_buckets:
            table = self._aux("rel", x.device, lambda: self.rel_bias.detach().float().contiguous())
            starts = self._aux("starts", x.device, lambda: torch.tensor(
                mops.log_bucket_starts(sp.bias_buckets, sp.bias_max), dtype=torch.int32))
            lut = self._aux("lut", x.device, lambda: mops.bucket_lut(
                mops.log_bucket_starts(sp.bias_buckets, sp.bias_max)))
        sinks = self._aux("sink", x.device, lambda: self.sink_logit.detach().float()) if sp.sink_learned else None
        slopes = self._aux("slopes", x.device, lambda: mops.distance_slopes(H)) if sp.dist_slopes else None
        o = kv_cache.attend_ragged(self.layer_idx, q, k, v, self.scale, bias_table=table, bucket_starts=starts,
                                   sink=sp.sink or sp.sink_learned, v_other=v_other, lam=lam, lut=lut,
                                   mask_block=sp.mask_block, wide_weights=sp.wide_weights, sink_values=sinks,
                                   slopes=slopes, window=sp.window)
        if sp.out_gate:
            o = mops.sigmoid_gate_mul(o, gate)
        return self.o_proj(o)


class LightningAttention(_MixerBase):
    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        H, d, dv = spec.heads, spec.dim, spec.vdim
        assert spec.decay is not None and len(spec.decay) == H, "one decay per head"
        self.in_proj = nn.Linear(cfg.hidden_size, 2 * H * d + 2 * H * dv, bias=False)      # q | k | v | gate
        self.norm_weight = nn.Parameter(torch.ones(H * dv))
        self.o_proj = nn.Linear(H * dv, cfg.hidden_size, bias=False)

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp = self.spec
        H, d, dv = sp.heads, sp.dim, sp.vdim
        z = self.in_proj(x)
        q, k, v, g = z.split([H * d, H * d, H * dv, H * dv], dim=-1)
        decay = self._aux("decay", x.device, lambda: torch.tensor(sp.decay, dtype=torch.float64).float())
        st = kv_cache.layer_state(self.layer_idx)
        o = mops.state_scan_decay(q, k, v, decay, st["S"], kv_cache.ragged, H, d, dv, act_silu=True)
        o = mops.gated_group_rms_norm(o, self.norm_weight, g, H * dv, self.cfg.norm_eps, x.dtype)
        return self.o_proj(o)


class ChannelDeltaMixer(_MixerBase):
    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        H, G, d, dv = spec.heads, spec.kv_heads, spec.dim, spec.vdim
        self.conv_channels = 2 * G * d + H * dv
        # q | k | v | write strength | decay bottleneck | gate bottleneck: one GEMM reads the layer input
        self.in_proj = nn.Linear(cfg.hidden_size, self.conv_channels + H + spec.decay_rank + spec.gate_rank, bias=False)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_channels, max(spec.conv, 1)))
        self.decay_up = nn.Linear(spec.decay_rank, H * d, bias=False)
        self.gate_up = nn.Linear(spec.gate_rank, H * dv, bias=False)
        self.A_log = nn.Parameter(torch.zeros(H))
        self.dt_bias = nn.Parameter(torch.zeros(H * d))
        self.norm_weight = nn.Parameter(torch.ones(dv))
        self.o_proj = nn.Linear(H * dv, cfg.hidden_size, bias=False)

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp = self.spec
        H, G, d, dv = sp.heads, sp.kv_heads, sp.dim, sp.vdim
        z = self.in_proj(x)
        qkv, b, a1, g1 = z.split([self.conv_channels, H, sp.decay_rank, sp.gate_rank], dim=-1)
        st = kv_cache.layer_state(self.layer_idx)
        ragged = kv_cache.ragged
        qkv = mops.short_conv_silu(qkv, self.conv_weight, st["conv"], ragged)
        q, k, v = qkv.split([G * d, G * d, H * dv], dim=-1)
        a = self.decay_up(a1)
        gate = self.gate_up(g1)
        a_log = self._aux("A_log", x.device, lambda: self.A_log.detach().float())
        dt_bias = self._aux("dt_bias", x.device, lambda: self.dt_bias.detach().float())
        o = mops.state_scan_delta(q, k, v, a, b, a_log, dt_bias, st["S"], ragged, H, G, d, dv)
        o = mops.gated_group_rms_norm(o, self.norm_weight, gate, dv, self.cfg.norm_eps, x.dtype)
        return self.o_proj(o)


class DeltaMixer(_MixerBase):
    """Gated delta rule with one decay per head.  W_in h = [q | k | v | write strength | decay | gate]; q | k | v pass a
    causal convolution and silu; q, k become unit vectors per head (q also times dim^-1/2); per token and head
    g = exp(-exp(A_log) softplus(a + dt_bias)), beta = sigmoid(b): S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  S [dim, vdim] is zero at the start of a sequence and carried in fp32 together with the convolution's last
    inputs.  Every head's o is divided by its root mean square, multiplied by a weight over vdim that the heads share and
    by silu(W_g h), and projected."""

    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        H, G, d, dv = spec.heads, spec.kv_heads, spec.dim, spec.vdim
        self.conv_channels = 2 * G * d + H * dv
        self.in_proj = nn.Linear(cfg.hidden_size, self.conv_channels + 2 * H + H * dv, bias=False)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_channels, max(spec.conv, 1)))
        self.A_log = nn.Parameter(torch.zeros(H))
        self.dt_bias = nn.Parameter(torch.zeros(H))
        self.norm_weight = nn.Parameter(torch.ones(dv))
        self.o_proj = nn.Linear(H * dv, cfg.hidden_size, bias=False)

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp = self.spec
        H, G, d, dv = sp.heads, sp.kv_heads, sp.dim, sp.vdim
        z = self.in_proj(x)
        qkv, b, a, gate = z.split([self.conv_channels, H, H, H * dv], dim=-1)
        st = kv_cache.layer_state(self.layer_idx)
        ragged = kv_cache.ragged
        qkv = mops.short_conv_silu(qkv, self.conv_weight, st["conv"], ragged)
        q, k, v = qkv.split([G * d, G * d, H * dv], dim=-1)
        a_log = self._aux("A_log", x.device, lambda: self.A_log.detach().float())
        dt_bias = self._aux("dt_bias", x.device, lambda: self.dt_bias.detach().float())
        o = mops.state_scan_delta(q, k, v, a, b, a_log, dt_bias, st["S"], ragged, H, G, d, dv, head_decay=True)
        o = mops.gated_group_rms_norm(o, self.norm_weight, gate, dv, self.cfg.norm_eps, x.dtype, gate_act="silu")
        return self.o_proj(o)


class LatentAttention(_MixerBase):
    """q = W_q h, per head [dim unrotated | rot_dim rotated]; W_dkv h = [kv_rank latent | rot_dim key part]; the latent is
    RMS-normalised (weight `dkv_norm_weight`) -> c, the key part is rotated -> k_r (one for all heads).  Head n scores
    position j with scale * (q_n . (U_n c_j) + q_r . k_r_j) and mixes the values V_n c_j.

    The cache holds one row [c | k_r] per token.  Both up-projections are absorbed into the query / output side:
    q_n . (U_n c) = (U_n^T q_n) . c, and sum_j p_j V_n c_j = V_n (sum_j p_j c_j), so the step runs multi-query attention
    with queries [U_n^T q_n | rotated q_r] against the cached rows, values = the rows' latent columns, and maps the
    `kv_rank`-wide results through V_n afterwards (two batched GEMMs over the heads).  A prompt, a portion and a decoded
    token take the same path, so a position's result does not depend on how the prompt was cut.

    Options of the spec: `q_rank` > 0 - the queries come through a latent of their own, q = W_uq (rms(W_dq h) w_dq) (the
    down-projection shares the GEMM that reads the layer input); `window` - a position sees the last `window` positions;
    `sink_learned` - a learned score per head joins the softmax's denominator; `rot_scaling` - stretched rotary
    frequencies (`ops.mixers.rotary_frequencies`)."""

    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        H, d, r, dv, R = spec.heads, spec.dim, spec.rot_dim, spec.vdim, spec.kv_rank
        assert spec.rot_dims in (0, r) and r % 2 == 0, "the decoupled key part is rotated as a whole"
        self.q_width = spec.q_rank or H * (d + r)
        self.in_proj = nn.Linear(cfg.hidden_size, self.q_width + R + r, bias=False)      # q (or its latent) | latent | key part
        if spec.q_rank:
            self.dq_norm_weight = nn.Parameter(torch.ones(spec.q_rank))
            self.uq_proj = nn.Linear(spec.q_rank, H * (d + r), bias=False)
        if spec.sink_learned:
            self.sink_logit = nn.Parameter(torch.zeros(H))
        self.dkv_norm_weight = nn.Parameter(torch.ones(R))
        self.uk = nn.Parameter(torch.empty(H, d, R))              # U_n: latent -> unrotated key of head n
        self.uv = nn.Parameter(torch.empty(H, dv, R))             # V_n: latent -> value of head n
        nn.init.normal_(self.uk, std=cfg.initializer_range)
        nn.init.normal_(self.uv, std=cfg.initializer_range)
        self.o_proj = nn.Linear(H * dv, cfg.hidden_size, bias=False)
        self.scale = spec.scale if spec.scale is not None else (d + r) ** -0.5

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp = self.spec
        H, d, r, dv, R = sp.heads, sp.dim, sp.rot_dim, sp.vdim, sp.kv_rank
        T = x.shape[0]
        z = self.in_proj(x)
        q, dkv = z[:, : self.q_width], z[:, self.q_width:]
        if sp.q_rank:
            q = self.uq_proj(mops.head_rms_norm(q, 1, 0, sp.q_rank, self.dq_norm_weight, None, self.cfg.norm_eps))
        ragged = kv_cache.ragged
        table = mops.rotary_table(kv_cache.max_len_host, r, sp.rot_base, x.device, sp.rot_scaling)
        mops.latent_kv_write(dkv, self.dkv_norm_weight, self.cfg.norm_eps, R, table, kv_cache.latent_cache(self.layer_idx),
                             kv_cache.block_tables, ragged)
        qa = torch.empty(T, H * (R + r), dtype=x.dtype, device=x.device)
        qa3 = qa.view(T, H, R + r)
        torch.bmm(q.view(T, H, d + r)[..., :d].transpose(0, 1), self.uk, out=qa3[..., :R].transpose(0, 1))
        mops.rotary_half(q, qa, H, d + r, d, R + r, R, r, r, table, ragged.token_pos)
        sinks = self._aux("sink", x.device, lambda: self.sink_logit.detach().float()) if sp.sink_learned else None
        o = kv_cache.attend_latent(self.layer_idx, qa, self.scale, R, window=sp.window,
                                   sink=sp.sink or sp.sink_learned, sink_values=sinks,
                                   wide_weights=sp.wide_weights)                              # [T, H x R]
        o = torch.bmm(o.view(T, H, R).transpose(0, 1), self.uv.transpose(1, 2))        # [H, T, dv]
        return self.o_proj(o.transpose(0, 1).reshape(T, H * dv))


class Retention(_MixerBase):
    """Per head a matrix S [dim, vdim], zero at the start of a sequence and carried in fp32: S <- decay_n S + outer(k, v),
    read-out S^T q after the write.  q, k get rotary positions on their first `rot_dims` channels and k the factor
    dim^-1/2, both in fp32; every head's read-out is divided by its root mean square (no weight), multiplied by
    silu(W_g h) and projected."""

    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        H, d, dv = spec.heads, spec.dim, spec.vdim
        assert spec.decay is not None and len(spec.decay) == H, "one decay per head"
        assert spec.rot_dims % 2 == 0 and spec.rot_dims <= d
        self.in_proj = nn.Linear(cfg.hidden_size, 2 * H * d + 2 * H * dv, bias=False)      # q | k | v | gate
        self.o_proj = nn.Linear(H * dv, cfg.hidden_size, bias=False)

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp = self.spec
        H, d, dv = sp.heads, sp.dim, sp.vdim
        z = self.in_proj(x)
        q, k, v, g = z.split([H * d, H * d, H * dv, H * dv], dim=-1)
        decay = self._aux("decay", x.device, lambda: torch.tensor(sp.decay, dtype=torch.float64).float())
        table = mops.rotary_table(kv_cache.max_len_host, sp.rot_dims, sp.rot_base, x.device) if sp.rot_dims else None
        st = kv_cache.layer_state(self.layer_idx)
        o = mops.state_scan_decay(q, k, v, decay, st["S"], kv_cache.ragged, H, d, dv, act_silu=False, rot_table=table,
                                  rot_dims=sp.rot_dims, k_scale=d ** -0.5)
        o = mops.gated_group_rms_norm(o, None, g, dv, self.cfg.norm_eps, x.dtype, gate_act="silu")
        return self.o_proj(o)


class MatrixLSTM(_MixerBase):
    """Per head a matrix S [dim, vdim], a normaliser n [dim] and a running maximum m, all zero at the start of a sequence
    and carried in fp32.  With cap(z) = gate_cap tanh(z / gate_cap): i = cap(W_i h + b_i), f = logsigmoid(cap(W_f h + b_f)),
    m' = max(f + m, i), S <- exp(f + m - m') S + exp(i - m') outer(k, v), n likewise with k alone; the read-out
    S^T q / (max(|n . q|, exp(-m')) + 1e-6), q scaled by dim^-1/2, is brought to unit RMS per head, multiplied by a weight
    over all heads' channels and by sigmoid(W_g h), and projected."""

    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        H, d, dv = spec.heads, spec.dim, spec.vdim
        self.in_proj = nn.Linear(cfg.hidden_size, 2 * H * d + 2 * H * dv + 2 * H, bias=False)   # q | k | v | gate | i | f
        self.gate_bias = nn.Parameter(torch.zeros(2 * H))                                       # b_i | b_f
        self.norm_weight = nn.Parameter(torch.ones(H * dv))
        self.o_proj = nn.Linear(H * dv, cfg.hidden_size, bias=False)

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp = self.spec
        H, d, dv = sp.heads, sp.dim, sp.vdim
        z = self.in_proj(x)
        q, k, v, g, gates = z.split([H * d, H * d, H * dv, H * dv, 2 * H], dim=-1)
        bias = self._aux("gate_bias", x.device, lambda: self.gate_bias.detach().float())
        st = kv_cache.layer_state(self.layer_idx)
        o = mops.state_scan_mlstm(q, k, v, gates, bias, sp.gate_cap, st["S"], st["n"], st["m"], kv_cache.ragged, H, d, dv,
                                  q_scale=d ** -0.5)
        o = mops.gated_group_rms_norm(o, self.norm_weight, g, dv, self.cfg.norm_eps, x.dtype)
        return self.o_proj(o)


class SelectiveStateSpace(_MixerBase):
    """inner = heads x vdim channels, `state` rows per head, B / C shared by `groups` of heads.  W_in h = [z | x | B | C | dt];
    x | B | C pass a causal convolution (with bias) and silu; step = softplus(dt + dt_bias); per head
    S <- exp(-exp(A_log) step) S + step outer(B, x), y = S^T C + D x, S [state, vdim] zero at the start and carried in fp32
    together with the convolution's last inputs.  y silu(z) is RMS-normed in `norm_groups` parts, weighted and projected."""

    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        H, dv, N, G = spec.heads, spec.vdim, spec.state, spec.groups
        self.inner = H * dv
        assert H % G == 0 and self.inner % spec.norm_groups == 0
        self.conv_channels = self.inner + 2 * G * N
        self.in_proj = nn.Linear(cfg.hidden_size, self.inner + self.conv_channels + H, bias=False)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_channels, max(spec.conv, 1)))
        self.conv_bias = nn.Parameter(torch.zeros(self.conv_channels))
        self.dt_bias = nn.Parameter(torch.zeros(H))
        self.A_log = nn.Parameter(torch.zeros(H))
        self.D = nn.Parameter(torch.ones(H))
        self.norm_weight = nn.Parameter(torch.ones(self.inner))
        self.o_proj = nn.Linear(self.inner, cfg.hidden_size, bias=False)

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp = self.spec
        H, dv, N, G = sp.heads, sp.vdim, sp.state, sp.groups
        zz = self.in_proj(x)
        z, xbc, dt = zz.split([self.inner, self.conv_channels, H], dim=-1)
        st = kv_cache.layer_state(self.layer_idx)
        ragged = kv_cache.ragged
        xbc = mops.short_conv_silu(xbc, self.conv_weight, st["conv"], ragged, bias=self.conv_bias)
        xs, b, c = xbc.split([self.inner, G * N, G * N], dim=-1)
        f32 = lambda name: self._aux(name, x.device, lambda: getattr(self, name).detach().float())
        y = mops.state_scan_ssd(c, b, xs, dt, f32("dt_bias"), f32("A_log"), f32("D"), st["S"], ragged, H, G, N, dv)
        y = mops.gated_group_rms_norm(y, self.norm_weight, z, self.inner // sp.norm_groups, self.cfg.norm_eps, x.dtype,
                                      gate_act="silu", gate_first=True)
        return self.o_proj(y)


class GatedLinearRecurrence(_MixerBase):
    """Two branches of `lru_width` channels: y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x) (causal, per channel,
    with bias, no activation).  u is cut into `blocks` parts; in part b, r = sigmoid(A_b u_b + a_b), i = sigmoid(I_b u_b +
    i_b); log a = -lru_c r softplus(lam); S <- a S + sqrt(1 - a^2) i u per channel, zero at the start and carried in fp32
    together with the convolution's last inputs; the output is W_o (S y).  The gate matrices' products keep their fp32
    accumulators (no 16-bit rounding in front of the sigmoids)."""

    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__(cfg, spec, layer_idx)
        C, nb = spec.lru_width, spec.blocks
        assert C % nb == 0
        bw = C // nb
        self.in_proj = nn.Linear(cfg.hidden_size, 2 * C, bias=True)                      # y branch | x branch
        self.conv_weight = nn.Parameter(torch.zeros(C, max(spec.conv, 1)))
        self.conv_bias = nn.Parameter(torch.zeros(C))
        self.gate_weight = nn.Parameter(torch.zeros(nb, 2 * bw, bw))                     # per block: recurrence gate | input gate
        self.gate_bias = nn.Parameter(torch.zeros(nb, 2 * bw))
        self.lam = nn.Parameter(torch.zeros(C))
        self.o_proj = nn.Linear(C, cfg.hidden_size, bias=False)
        nn.init.normal_(self.gate_weight, std=cfg.initializer_range)

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        sp = self.spec
        C, nb = sp.lru_width, sp.blocks
        T = x.shape[0]
        z = self.in_proj(x)
        branch, xb = z[:, :C], z[:, C:]
        st = kv_cache.layer_state(self.layer_idx)
        ragged = kv_cache.ragged
        u = mops.short_conv_silu(xb, self.conv_weight, st["conv"], ragged, activation=False, bias=self.conv_bias)
        ub = u.view(T, nb, C // nb).transpose(0, 1)                                      # [blocks, T, bw]
        wt = self.gate_weight.transpose(1, 2)                                            # [blocks, bw, 2 bw]
        if u.is_cuda and u.dtype != torch.float32:
            gates = torch.bmm(ub, wt, out_dtype=torch.float32)
        else:
            gates = torch.bmm(ub.float(), wt.float())
        f32 = lambda name: self._aux(name, x.device, lambda: getattr(self, name).detach().float().contiguous())
        s = mops.lru_scan(u, gates.contiguous(), f32("gate_bias"), f32("lam"), branch, st["S"], ragged, c=sp.lru_c)
        return self.o_proj(s)


class MixerPair(nn.Module):
    """Mixers side by side: every part reads the same input, its output is RMS-normed over the model width with a plain
    weight of its own, and the results are averaged (in fp32: the sum goes straight into the residual stream).  The paged
    part uses the layer's pages, the recurrent part the layer's state slot."""

    def __init__(self, cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> None:
        super().__init__()
        self.cfg, self.spec, self.layer_idx = cfg, spec, layer_idx
        self.shard_config = None
        self.parts = nn.ModuleList([_build(cfg, p, layer_idx) for p in spec.parts])
        self.out_norm_weights = nn.ParameterList([nn.Parameter(torch.ones(cfg.hidden_size)) for _ in spec.parts])

    def forward(self, x: torch.Tensor, meta, rope=None, kv_cache=None) -> torch.Tensor:
        outs = [m(x, meta, rope, kv_cache) for m in self.parts]
        return mops.norm_mean(outs, list(self.out_norm_weights), self.cfg.norm_eps)


_KINDS = {"attention": BiasSinkAttention, "lightning": LightningAttention, "channel_delta": ChannelDeltaMixer,
          "latent": LatentAttention, "retention": Retention, "mlstm": MatrixLSTM, "ssd": SelectiveStateSpace,
          "rglru": GatedLinearRecurrence, "pair": MixerPair, "delta": DeltaMixer}


def _build(cfg: ModelConfig, spec: MixerSpec, layer_idx: int) -> nn.Module:
    if spec.kind not in _KINDS:
        raise ValueError(f"unknown mixer kind {spec.kind!r}; known: {sorted(_KINDS)}")
    return _KINDS[spec.kind](cfg, spec, layer_idx)


def build_mixer(cfg: ModelConfig, layer_idx: int) -> nn.Module:
    return _build(cfg, cfg.layer_specs[layer_idx].mixer, layer_idx)
