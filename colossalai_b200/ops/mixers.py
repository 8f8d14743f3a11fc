"""Python face of the sequence-mixer kernels (kernel/csrc/mixers.cu): short causal convolution with a carried window,
recurrent state scans (decayed outer-product state with optional rotary positions, gated delta rule, per-token gated
outer-product state for selective state spaces and the exponentially gated matrix memory, per-channel gated linear
recurrence), group RMS norm with a sigmoid / silu gate before or after the norm, rotary positions + unit norm of q / k
heads, the mean of RMS-normed mixer outputs, RMS norm of a sublayer's output added to an fp32 residual stream, sums into the fp32 stream
fused with the next RMS / layer norm, rotary positions from an fp32 angle table, the cache rows of latent attention, and
paged attention with a distance-bucket bias and a softmax sink (values optionally read from the key rows).

All ops take a RAGGED step (`RaggedMeta`): for every live sequence its next tokens, how many tokens earlier steps
consumed, and the slot that holds its carried state.  CUDA tensors go to the sm_100a kernels; CPU tensors take the plain
PyTorch path below (the plumbing tier of the test-suite), which follows the same token-by-token order.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..kernel import loader
from ._dispatch import use_native
from ._dtypes import code

__all__ = ["RaggedMeta", "short_conv_silu", "state_scan_decay", "state_scan_delta", "gated_group_rms_norm",
           "rms_norm_residual", "rms_norm_f32in", "paged_kv_write_mix", "paged_bias_attention", "log_bucket_starts",
           "bucket_lut", "rotary_table", "rotary_half", "stream_add_norm", "latent_kv_write", "state_scan_ssd",
           "state_scan_mlstm", "lru_scan", "rotary_unit_norm", "sigmoid_gate_mul", "norm_mean", "depth_mix", "poly_norm",
           "head_rms_norm", "distance_slopes"]

_lib = None
_SPLIT_BELOW_TILES = 148        # attention steps with fewer CTAs than SMs split their keys


def _get_lib():
    global _lib
    if _lib is None:
        _lib = loader.load("cb200_mixers")
        _lib.cb_state_scan_workspace.restype = ctypes.c_int64
    return _lib


_workspaces = {}


def _workspace(name: str, numel: int, device) -> torch.Tensor:
    """Grow-only fp32 scratch per (purpose, device): consecutive layers run on one stream, so they can share it."""
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        # a captured step keeps its own scratch in the graph's pool: the shared one may be regrown (freed) later
        return torch.empty(max(int(numel), 1), dtype=torch.float32, device=device)
    key = (name, str(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(int(numel), 1), dtype=torch.float32, device=device)
        _workspaces[key] = buf
    return buf


def _i64(v: int) -> ctypes.c_int64:
    return ctypes.c_int64(int(v))


def _f(v: float) -> ctypes.c_float:
    return ctypes.c_float(float(v))


@dataclass
class RaggedMeta:
    """One step's layout.  Device tensors are int32; the python lists mirror them so no op has to synchronise."""

    cu_q: torch.Tensor            # [nseq + 1] first flat token of every sequence's portion
    ctx_len: torch.Tensor         # [nseq] tokens consumed by earlier steps
    slots: torch.Tensor           # [nseq] state slot of the sequence
    token_seq: torch.Tensor       # [T] sequence index of every token
    token_pos: torch.Tensor       # [T] position of every token in its sequence
    q_lens: List[int]
    ctx_lens: List[int]
    slot_list: List[int]

    @property
    def nseq(self) -> int:
        return len(self.q_lens)

    @property
    def max_q(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @staticmethod
    def layout(flat: torch.Tensor, nseq: int, tokens: int):
        """Views of one flat int32 buffer [cu_q | ctx_len | slots | token_seq | token_pos]."""
        a, b, c, d = nseq + 1, 2 * nseq + 1, 3 * nseq + 1, 3 * nseq + 1 + tokens
        return flat[:a], flat[a:b], flat[b:c], flat[c:d], flat[d:d + tokens]

    @staticmethod
    def flat_list(q_lens: Sequence[int], ctx_lens: Sequence[int], slots: Sequence[int]) -> List[int]:
        cu, seq, pos = [0], [], []
        for i, (n, c) in enumerate(zip(q_lens, ctx_lens)):
            cu.append(cu[-1] + int(n))
            seq += [i] * int(n)
            pos += range(int(c), int(c) + int(n))
        return cu + [int(c) for c in ctx_lens] + [int(x) for x in slots] + seq + pos

    @staticmethod
    def decode_static(flat: torch.Tensor, nseq: int, max_ctx: int) -> "RaggedMeta":
        """One token per sequence over a fixed device buffer (CUDA-graph replay refills `flat`): the host-side mirror
        holds the worst case (`max_ctx` cached tokens) so that launch shapes do not depend on the step."""
        cu, ctx, slots, seq, pos = RaggedMeta.layout(flat, nseq, nseq)
        return RaggedMeta(cu, ctx, slots, seq, pos, [1] * nseq, [max_ctx] * nseq, list(range(nseq)))

    @staticmethod
    def build(q_lens: Sequence[int], ctx_lens: Sequence[int], slots: Sequence[int], device) -> "RaggedMeta":
        q_lens, ctx_lens, slots = [int(x) for x in q_lens], [int(x) for x in ctx_lens], [int(x) for x in slots]
        cu = [0]
        seq, pos = [], []
        for i, (n, c) in enumerate(zip(q_lens, ctx_lens)):
            cu.append(cu[-1] + n)
            seq += [i] * n
            pos += range(c, c + n)
        flat = torch.tensor(cu + ctx_lens + slots + seq + pos, dtype=torch.int32).to(device, non_blocking=True)
        n = len(q_lens)
        a, b, c, d = n + 1, 2 * n + 1, 3 * n + 1, 3 * n + 1 + len(seq)
        return RaggedMeta(flat[:a], flat[a:b], flat[b:c], flat[c:d], flat[d:], q_lens, ctx_lens, slots)


def log_bucket_starts(num_buckets: int, max_distance: float) -> List[int]:
    """Smallest distance that falls into every bucket of a table whose first half is exact and whose second half is
    logarithmic up to `max_distance`.  With h = B // 2 rows for the exact part, a distance below h is its own row and
    a distance n >= h lands in row h + floor((B - h) * log(n / h) / log(max_distance / h)), clipped to the last row."""
    B, half = num_buckets, num_buckets // 2

    def bucket(n: int) -> int:
        if n < half:
            return n
        return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(max_distance / half) * (B - half))))

    starts = list(range(half)) + [0] * (B - half)
    n = half
    for b in range(half, B):
        while bucket(n) < b:
            n += 1
        starts[b] = n
    return starts


def bucket_lut(starts: Sequence[int]) -> torch.Tensor:
    """distance -> bucket for every distance below the last bucket's first one (uint8; larger distances fall into the
    last bucket), the form the tensor-core attention kernel reads."""
    starts = [int(x) for x in starts]
    lut = torch.zeros(max(starts[-1], 1), dtype=torch.uint8)
    for b in range(len(starts) - 1):
        lut[starts[b]: starts[b + 1]] = b
    return lut


# ------------------------------------------------------------------------------------------------ rotary positions
_rotary_tables = {}


def rotary_frequencies(dims: int, base: float, scaling: Optional[Sequence[float]] = None):
    """(f [dims / 2] float64, factor on cos / sin).  f_i = base^(-2 i / dims).  `scaling` = (s, n, fast, slow) stretches
    the slow frequencies for contexts beyond the n positions the model was trained on: with
    d(t) = dims ln(n / (2 pi t)) / (2 ln base) - the channel that turns t times over n positions - lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency becomes
    f_i / s * r_i + f_i * (1 - r_i), and cos and sin are multiplied by 0.1 ln(s) + 1."""
    f = torch.tensor(float(base), dtype=torch.float64) ** (-torch.arange(0, dims, 2, dtype=torch.float64) / dims)
    if not scaling:
        return f, 1.0
    s, n, fast, slow = [float(v) for v in scaling]
    d = lambda t: dims * math.log(n / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(d(fast)), 0)
    hi = min(math.ceil(d(slow)), dims - 1)
    r = ((torch.arange(dims // 2, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / s * r + f * (1.0 - r), 0.1 * math.log(s) + 1.0


def rotary_table(min_len: int, dims: int, base: float, device, scaling: Optional[Sequence[float]] = None) -> torch.Tensor:
    """fp32 [positions, dims]: row p holds c cos(p f_i) for i < dims / 2, then c sin(p f_i), with (f, c) =
    `rotary_frequencies(dims, base, scaling)`.  Angles are formed in float64 and rounded once.  The table is cached per
    (dims, base, scaling, device) and grows in powers of two, so that positions far beyond any configured length stay
    exact."""
    key = (int(dims), float(base), tuple(float(v) for v in scaling) if scaling else None, str(device))
    tab = _rotary_tables.get(key)
    if tab is None or tab.shape[0] < min_len:
        n = max(1024, 1 << max(int(min_len) - 1, 1).bit_length())
        f, c = rotary_frequencies(dims, base, scaling)
        ang = torch.arange(n, dtype=torch.float64)[:, None] * f[None, :]
        tab = (torch.cat([ang.cos(), ang.sin()], 1) * c).float().to(device)
        _rotary_tables[key] = tab
    return tab


def distance_slopes(heads: int) -> torch.Tensor:
    """fp32 [heads]: 2^(-8 (h + 1) / heads), the per-head slope of a linear distance penalty."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float64).float()


def _rot_ref(x: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, H, w] fp32: channel i < dims / 2 of every head is paired with channel i + dims / 2."""
    half = dims // 2
    cs = table[pos.long()]
    c, sn = cs[:, None, :half], cs[:, None, half:]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * sn, v * c + u * sn, x[..., dims:]], -1)


def rotary_half(src: torch.Tensor, dst: torch.Tensor, heads: int, src_head_stride: int, src_off: int,
                dst_head_stride: int, dst_off: int, width: int, dims: int, table: torch.Tensor,
                token_pos: torch.Tensor) -> None:
    """For every token t and head h: dst[t, h * dst_head_stride + dst_off + (0..width)] = the `width` channels at
    src[t, h * src_head_stride + src_off + ..] with the first `dims` of them turned by the token's position (rotate-half
    pairs, fp32 arithmetic, one rounding into dst's dtype)."""
    T = src.shape[0]
    if use_native(src):
        assert src.stride(1) == 1 and dst.stride(1) == 1 and table.dtype == torch.float32 and table.shape[1] == dims
        loader.check(_get_lib().cb_rotary_half(
            loader.ptr(src), _i64(src.stride(0)), loader.ptr(dst), _i64(dst.stride(0)), _i64(T), heads, src_head_stride,
            src_off, dst_head_stride, dst_off, width, dims, loader.ptr(table), loader.ptr(token_pos), code(src.dtype),
            code(dst.dtype), loader.stream_ptr()), "rotary_half")
        loader.launch_counter.add("rotary_half")
        return
    cols = (torch.arange(heads)[:, None] * src_head_stride + src_off + torch.arange(width)[None, :]).reshape(-1)
    x = src[:, cols].float().view(T, heads, width)
    y = _rot_ref(x, token_pos, table, dims)
    dcols = (torch.arange(heads)[:, None] * dst_head_stride + dst_off + torch.arange(width)[None, :]).reshape(-1)
    dst[:, dcols] = y.reshape(T, heads * width).to(dst.dtype)


# ------------------------------------------------------------------------------------------------ short convolution
def short_conv_silu(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, meta: RaggedMeta,
                    activation: bool = True, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C] (may be a column slice, unit stride inside a row); weight [C, taps], last column = current token;
    state [slots, taps - 1, C] = the last inputs of every sequence, read and advanced; `bias` [C] is added to the sum of
    the taps.  Returns silu(conv) (or the plain sum when `activation` is off) [T, C]."""
    T, C = x.shape
    taps = weight.shape[1]
    out = torch.empty(T, C, dtype=x.dtype, device=x.device)
    if use_native(x):
        assert x.stride(1) == 1 and weight.is_contiguous() and state.is_contiguous() and state.dtype == x.dtype
        assert bias is None or (bias.is_contiguous() and bias.dtype == x.dtype and bias.numel() == C)
        loader.check(_get_lib().cb_short_conv_silu(
            loader.ptr(x), _i64(x.stride(0)), loader.ptr(weight), loader.ptr(bias), loader.ptr(state), loader.ptr(out),
            _i64(C), loader.ptr(meta.cu_q), loader.ptr(meta.ctx_len), loader.ptr(meta.slots), meta.nseq, meta.max_q, C,
            taps, int(activation), 1, code(x.dtype), loader.stream_ptr()), "short_conv_silu")
        loader.launch_counter.add("short_conv_silu", 2)
        return out
    t0 = 0
    w = weight.float()
    for n, c, slot in zip(meta.q_lens, meta.ctx_lens, meta.slot_list):
        if n == 0:
            continue
        prev = state[slot].float() if c > 0 else torch.zeros(taps - 1, C)
        full = torch.cat([prev, x[t0:t0 + n].float()], 0)                     # [taps - 1 + n, C]
        acc = torch.zeros(n, C)
        for i in range(taps):
            acc += full[i:i + n] * w[:, i]
        if bias is not None:
            acc += bias.float()
        out[t0:t0 + n] = (F.silu(acc) if activation else acc).to(x.dtype)
        if taps > 1:
            state[slot] = full[n:].to(state.dtype)
        t0 += n
    return out


# ------------------------------------------------------------------------------------------------ state scans
def _scan_native(mode, q, k, v, araw, braw, head_decay, a_log, dt_bias, state, meta, heads, qk_heads, dim, vdim,
                 act_silu, unit_qk, unit_eps, q_scale, k_scale=1.0, rot_table=None, rot_dims=0, gate_cap=0.0,
                 gate_kind=0, state_n=None, state_m=None):
    T = q.shape[0]
    out = torch.empty(T, heads * vdim, dtype=torch.float32, device=q.device)
    for t in (q, k, v):
        assert t.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous()
    ld = lambda t: _i64(0 if t is None else t.stride(0))
    lib = _get_lib()
    # fp32 rows the elementwise prepare kernel writes and the recurrence streams through shared memory
    work = _workspace("scan", lib.cb_state_scan_workspace(mode, _i64(T), heads, qk_heads, dim, vdim), q.device)
    loader.check(lib.cb_state_scan(
        mode, loader.ptr(q), ld(q), loader.ptr(k), ld(k), loader.ptr(v), ld(v), loader.ptr(araw), ld(araw),
        loader.ptr(braw), ld(braw), loader.ptr(head_decay), loader.ptr(a_log), loader.ptr(dt_bias), loader.ptr(state),
        loader.ptr(out), loader.ptr(work), _i64(T), loader.ptr(meta.cu_q), loader.ptr(meta.ctx_len),
        loader.ptr(meta.slots), meta.nseq, heads, qk_heads, dim, vdim, int(act_silu), int(unit_qk), _f(unit_eps),
        _f(q_scale), _f(k_scale), loader.ptr(rot_table), int(rot_dims if rot_table is not None else 0),
        loader.ptr(meta.token_pos), int(gate_kind), _f(gate_cap), loader.ptr(state_n), loader.ptr(state_m),
        code(q.dtype), loader.stream_ptr()), "state_scan")
    loader.launch_counter.add("state_scan", 3 if gate_kind == 2 else 2)
    return out


def state_scan_decay(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, head_decay: torch.Tensor, state: torch.Tensor,
                     meta: RaggedMeta, heads: int, dim: int, vdim: int, act_silu: bool = True,
                     rot_table: Optional[torch.Tensor] = None, rot_dims: int = 0, q_scale: float = 1.0,
                     k_scale: float = 1.0) -> torch.Tensor:
    """Decayed outer-product memory per head: every token scales the head's matrix M [dim, vdim] by the head's decay,
    adds outer(k, v) and reads y = M^T q (q, k, v through silu first when `act_silu`).  With `rot_table`
    (`rotary_table`) the first `rot_dims` channels of every q / k head are turned by the token's position, in fp32, before
    `q_scale` / `k_scale` multiply them.  q, k [T, heads x dim], v [T, heads x vdim]; state [slots, heads, dim, vdim] fp32.
    Returns fp32 o."""
    if dim > 256:
        raise NotImplementedError("state_scan: key width above 256 is not supported")
    if use_native(q):
        return _scan_native(0, q, k, v, None, None, head_decay, None, None, state, meta, heads, heads, dim, vdim,
                            act_silu, False, 0.0, q_scale, k_scale, rot_table, rot_dims)
    T = q.shape[0]
    out = torch.empty(T, heads * vdim, dtype=torch.float32)
    act = F.silu if act_silu else (lambda z: z)
    t0 = 0
    dec = head_decay.float()[:, None, None]
    for n, c, slot in zip(meta.q_lens, meta.ctx_lens, meta.slot_list):
        if n == 0:
            continue
        S = state[slot].clone() if c > 0 else torch.zeros_like(state[slot])
        qq = act(q[t0:t0 + n].float()).view(n, heads, dim)
        kk = act(k[t0:t0 + n].float()).view(n, heads, dim)
        vv = act(v[t0:t0 + n].float()).view(n, heads, vdim)
        if rot_table is not None and rot_dims > 0:
            qq = _rot_ref(qq, meta.token_pos[t0:t0 + n], rot_table, rot_dims)
            kk = _rot_ref(kk, meta.token_pos[t0:t0 + n], rot_table, rot_dims)
        qq, kk = qq * q_scale, kk * k_scale
        for t in range(n):
            S = dec * S + kk[t][:, :, None] * vv[t][:, None, :]
            out[t0 + t] = torch.einsum("hdv,hd->hv", S, qq[t]).reshape(-1)
        state[slot] = S
        t0 += n
    return out


def state_scan_delta(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay_pre: torch.Tensor, beta_pre: torch.Tensor,
                     a_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor, meta: RaggedMeta, heads: int,
                     qk_heads: int, dim: int, vdim: int, unit_eps: float = 1e-6,
                     q_scale: Optional[float] = None, head_decay: bool = False) -> torch.Tensor:
    """Gated delta rule with one decay per head and key channel.  Per token and head: q, k -> unit vectors (q also times
    `q_scale`), row decays r = exp(-exp(a_log_h) * softplus(decay_pre + dt_bias)), write strength w = sigmoid(beta_pre);
    the head's matrix M [dim, vdim] is first decayed row by row (M <- diag(r) M), then corrected towards v along k
    (e = w * (v - M^T k); M <- M + outer(k, e)) and read after the write (y = M^T q).  q, k [T, qk_heads x dim] (head h reads
    h // (heads / qk_heads)), v [T, heads x vdim], decay_pre [T, heads x dim], beta_pre [T, heads]; fp32 state.
    With `head_decay` the decay is ONE number per head and token: decay_pre [T, heads], dt_bias [heads]."""
    if dim > 256:
        raise NotImplementedError("state_scan: key width above 256 is not supported")
    q_scale = dim ** -0.5 if q_scale is None else q_scale
    if use_native(q):
        assert decay_pre.stride(1) == 1 and beta_pre.stride(1) == 1
        return _scan_native(1, q, k, v, decay_pre, beta_pre, None, a_log, dt_bias, state, meta, heads, qk_heads, dim,
                            vdim, False, True, unit_eps, q_scale, gate_kind=3 if head_decay else 0)
    T = q.shape[0]
    out = torch.empty(T, heads * vdim, dtype=torch.float32)
    rep = heads // qk_heads
    A = a_log.float().exp()[None, :, None]
    t0 = 0
    for n, c, slot in zip(meta.q_lens, meta.ctx_lens, meta.slot_list):
        if n == 0:
            continue
        S = state[slot].clone() if c > 0 else torch.zeros_like(state[slot])
        qq = q[t0:t0 + n].float().view(n, qk_heads, dim)
        kk = k[t0:t0 + n].float().view(n, qk_heads, dim)
        qq = qq / torch.sqrt((qq * qq).sum(-1, keepdim=True) + unit_eps) * q_scale
        kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + unit_eps)
        qq, kk = qq.repeat_interleave(rep, 1), kk.repeat_interleave(rep, 1)
        vv = v[t0:t0 + n].float().view(n, heads, vdim)
        gd = 1 if head_decay else dim
        g = torch.exp(-A * _softplus(decay_pre[t0:t0 + n].float().view(n, heads, gd)
                                     + dt_bias.float().view(1, heads, gd)))
        beta = torch.sigmoid(beta_pre[t0:t0 + n].float())
        for t in range(n):
            S = g[t][:, :, None] * S
            u = beta[t][:, None] * (vv[t] - torch.einsum("hdv,hd->hv", S, kk[t]))
            S = S + kk[t][:, :, None] * u[:, None, :]
            out[t0 + t] = torch.einsum("hdv,hd->hv", S, qq[t]).reshape(-1)
        state[slot] = S
        t0 += n
    return out


def _softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 20.0, x, torch.log1p(torch.exp(torch.clamp(x, max=20.0))))


def state_scan_ssd(c: torch.Tensor, b: torch.Tensor, x: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor,
                   a_log: torch.Tensor, skip: torch.Tensor, state: torch.Tensor, meta: RaggedMeta, heads: int,
                   groups: int, dim: int, vdim: int) -> torch.Tensor:
    """Selective state space, one matrix S [dim, vdim] per head.  Per token and head h (group g = h // (heads / groups)):
    step = softplus(dt_h + dt_bias_h); S <- exp(-exp(a_log_h) * step) S + step * outer(b_g, x_h); y_h = S^T c_g + skip_h x_h.
    c, b [T, groups x dim], x [T, heads x vdim], dt [T, heads] (any float dtype; steps, decays and S are fp32);
    dt_bias, a_log, skip [heads] fp32; state [slots, heads, dim, vdim] fp32.  Returns fp32 y [T, heads x vdim]."""
    if dim > 256:
        raise NotImplementedError("state_scan: key width above 256 is not supported")
    if use_native(x):
        return _scan_native(2, c, b, x, dt, None, skip, a_log, dt_bias, state, meta, heads, groups, dim, vdim,
                            False, False, 0.0, 1.0, gate_kind=1)
    T = x.shape[0]
    out = torch.empty(T, heads * vdim, dtype=torch.float32)
    rep = heads // groups
    A = a_log.float().exp()
    t0 = 0
    for n, ctx, slot in zip(meta.q_lens, meta.ctx_lens, meta.slot_list):
        if n == 0:
            continue
        S = state[slot].clone() if ctx > 0 else torch.zeros_like(state[slot])
        cc = c[t0:t0 + n].float().view(n, groups, dim).repeat_interleave(rep, 1)
        bb = b[t0:t0 + n].float().view(n, groups, dim).repeat_interleave(rep, 1)
        xx = x[t0:t0 + n].float().view(n, heads, vdim)
        step = _softplus(dt[t0:t0 + n].float() + dt_bias.float())
        dec = torch.exp(-A * step)
        for t in range(n):
            S = dec[t][:, None, None] * S + bb[t][:, :, None] * (step[t][:, None] * xx[t])[:, None, :]
            out[t0 + t] = (torch.einsum("hdv,hd->hv", S, cc[t]) + skip.float()[:, None] * xx[t]).reshape(-1)
        state[slot] = S
        t0 += n
    return out


def state_scan_mlstm(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gates: torch.Tensor, gate_bias: torch.Tensor,
                     gate_cap: float, state: torch.Tensor, state_n: torch.Tensor, state_m: torch.Tensor,
                     meta: RaggedMeta, heads: int, dim: int, vdim: int, q_scale: float,
                     den_eps: float = 1e-6) -> torch.Tensor:
    """Matrix memory with exponential gates.  gates [T, 2 x heads] = pre-activations of the input gate, then of the
    forget gate; gate_bias [2 x heads] fp32.  With cap(z) = gate_cap * tanh(z / gate_cap) (identity when gate_cap is 0):
    i = cap(gates_i + bias_i), f = logsigmoid(cap(gates_f + bias_f)); m' = max(f + m, i);
    S <- exp(f + m - m') S + exp(i - m') outer(k, v), n likewise with k alone, m <- m';
    y = S^T q / (max(|n . q|, exp(-m)) + den_eps) with q scaled by `q_scale`.  S, n and m start at zero and are carried
    in fp32 (state [slots, heads, dim, vdim], state_n [slots, heads, dim], state_m [slots, heads]).  Returns fp32 y."""
    if dim > 256:
        raise NotImplementedError("state_scan: key width above 256 is not supported")
    if use_native(q):
        assert gates.stride(1) == 1 and state_n.is_contiguous() and state_m.is_contiguous()
        assert abs(den_eps - 1e-6) < 1e-12, "the kernel holds the denominator's floor at 1e-6"
        return _scan_native(2, q, k, v, gates, None, None, None, gate_bias, state, meta, heads, heads, dim, vdim,
                            False, False, 0.0, q_scale, gate_cap=gate_cap, gate_kind=2, state_n=state_n,
                            state_m=state_m)
    T = q.shape[0]
    out = torch.empty(T, heads * vdim, dtype=torch.float32)
    t0 = 0
    for cnt, ctx, slot in zip(meta.q_lens, meta.ctx_lens, meta.slot_list):
        if cnt == 0:
            continue
        S = state[slot].clone() if ctx > 0 else torch.zeros_like(state[slot])
        nn_ = state_n[slot].clone() if ctx > 0 else torch.zeros_like(state_n[slot])
        m = state_m[slot].clone() if ctx > 0 else torch.zeros_like(state_m[slot])
        qq = q[t0:t0 + cnt].float().view(cnt, heads, dim) * q_scale
        kk = k[t0:t0 + cnt].float().view(cnt, heads, dim)
        vv = v[t0:t0 + cnt].float().view(cnt, heads, vdim)
        z = gates[t0:t0 + cnt].float() + gate_bias.float()
        if gate_cap:
            z = gate_cap * torch.tanh(z / gate_cap)
        ig, fg = z[:, :heads], F.logsigmoid(z[:, heads:])
        for t in range(cnt):
            mn = torch.maximum(fg[t] + m, ig[t])
            a, w = torch.exp(fg[t] + m - mn), torch.exp(ig[t] - mn)
            S = a[:, None, None] * S + kk[t][:, :, None] * (w[:, None] * vv[t])[:, None, :]
            nn_ = a[:, None] * nn_ + w[:, None] * kk[t]
            m = mn
            den = torch.maximum((nn_ * qq[t]).sum(-1).abs(), torch.exp(-m)) + den_eps
            out[t0 + t] = (torch.einsum("hdv,hd->hv", S, qq[t]) / den[:, None]).reshape(-1)
        state[slot], state_n[slot], state_m[slot] = S, nn_, m
        t0 += cnt
    return out


def _gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z * z * z)))


def lru_scan(u: torch.Tensor, gates: torch.Tensor, gate_bias: torch.Tensor, lam: torch.Tensor, branch: torch.Tensor,
             state: torch.Tensor, meta: RaggedMeta, c: float = 8.0) -> torch.Tensor:
    """Gated linear recurrence per channel.  u [T, C]; gates [blocks, T, 2 x C / blocks] fp32 = pre-activations of the
    recurrence gate, then of the input gate, of every block's channels (without `gate_bias` [blocks, 2 x C / blocks]);
    lam [C] fp32; branch [T, C] = pre-activation of the multiplicative branch.  Per token:
    r = sigmoid(.), i = sigmoid(.), log a = -c r softplus(lam), S <- a S + sqrt(1 - a^2) i u, out = S * gelu_tanh(branch).
    S starts at zero and is carried in fp32 (state [slots, C]).  Returns [T, C] in u's dtype."""
    T, C = u.shape
    nb = gates.shape[0]
    bw = C // nb
    if use_native(u):
        assert gates.dtype == torch.float32 and gates.is_contiguous() and u.stride(1) == 1 and branch.stride(1) == 1
        assert state.dtype == torch.float32 and state.is_contiguous() and branch.dtype == u.dtype
        out = torch.empty(T, C, dtype=u.dtype, device=u.device)
        loader.check(_get_lib().cb_lru_scan(
            loader.ptr(u), _i64(u.stride(0)), loader.ptr(gates), loader.ptr(gate_bias), loader.ptr(lam),
            loader.ptr(branch), _i64(branch.stride(0)), loader.ptr(state), loader.ptr(out), _i64(T), loader.ptr(meta.cu_q),
            loader.ptr(meta.ctx_len), loader.ptr(meta.slots), meta.nseq, C, nb, _f(c), code(u.dtype),
            loader.stream_ptr()), "lru_scan")
        loader.launch_counter.add("lru_scan")
        return out
    out = torch.empty(T, C, dtype=u.dtype)
    g = (gates.float() + gate_bias.float()[:, None, :]).sigmoid()                 # [blocks, T, 2 bw]
    r = g[:, :, :bw].permute(1, 0, 2).reshape(T, C)
    ii = g[:, :, bw:].permute(1, 0, 2).reshape(T, C)
    loga = -c * r * _softplus(lam.float())
    a = torch.exp(loga)
    mult = torch.sqrt(-torch.expm1(2.0 * loga)) * ii * u.float()
    y = _gelu_tanh(branch.float())
    t0 = 0
    for n, ctx, slot in zip(meta.q_lens, meta.ctx_lens, meta.slot_list):
        if n == 0:
            continue
        S = state[slot].clone() if ctx > 0 else torch.zeros_like(state[slot])
        for t in range(t0, t0 + n):
            S = a[t] * S + mult[t]
            out[t] = (S * y[t]).to(u.dtype)
        state[slot] = S
        t0 += n
    return out


# ------------------------------------------------------------------------------------------------ norms
def gated_group_rms_norm(o: torch.Tensor, weight: Optional[torch.Tensor], gate: Optional[torch.Tensor], group: int,
                         eps: float, out_dtype: torch.dtype, gate_act: str = "sigmoid",
                         gate_first: bool = False) -> torch.Tensor:
    """o [T, C] fp32 -> o / sqrt(mean over each group of `group` channels + eps) * weight[c % len(weight)]
    * act(gate), in `out_dtype`; act is the sigmoid or (`gate_act="silu"`) the silu; without `weight` the norm is plain.
    With `gate_first` the gate multiplies o BEFORE the norm: (o act(gate)) / rms_group(o act(gate)) * weight."""
    T, C = o.shape
    assert gate_act in ("sigmoid", "silu") and not (gate_first and gate is None)
    if use_native(o):
        out = torch.empty(T, C, dtype=out_dtype, device=o.device)
        assert o.is_contiguous() and (weight is None or weight.dtype == out_dtype) and \
            (gate is None or (gate.stride(1) == 1 and gate.dtype == out_dtype))
        loader.check(_get_lib().cb_gated_group_rmsnorm(
            loader.ptr(o), loader.ptr(weight), 1 if weight is None else weight.numel(), loader.ptr(gate),
            _i64(0 if gate is None else gate.stride(0)), loader.ptr(out), _i64(T), C, group, _f(eps),
            int(gate_act == "silu") | (2 if gate_first else 0), code(out_dtype), loader.stream_ptr()),
            "gated_group_rmsnorm")
        loader.launch_counter.add("gated_group_rmsnorm")
        return out
    if gate_first:
        o = o * (torch.sigmoid(gate.float()) if gate_act == "sigmoid" else F.silu(gate.float()))
        gate = None
    y = o.view(T, C // group, group)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    y = y.reshape(T, C)
    if weight is not None:
        y = y * weight.float().repeat(C // weight.numel())
    if gate is not None:
        y = y * (torch.sigmoid(gate.float()) if gate_act == "sigmoid" else F.silu(gate.float()))
    return y.to(out_dtype)


def _group_rms(y: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    T, W = y.shape
    g = y.view(T, groups, W // groups)
    return (g / torch.sqrt((g * g).mean(-1, keepdim=True) + eps)).reshape(T, W)


def rms_norm_residual(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, mult: float = 1.0,
                      offset: float = 0.0, want_cast: bool = True, groups: int = 1,
                      history: Optional[tuple] = None) -> Optional[torch.Tensor]:
    """x [T, W] fp32, updated in place: x += mult * y / rms(y) * (offset + weight); with `groups` > 1 the row of y is cut
    into that many equal consecutive parts and each is divided by its own root mean square.  y is in the weight's dtype
    or fp32 (a sum kept in fp32).  Returns x in the weight's dtype.

    `history` = (hist [slices, T, W] fp32, n, coef [>= n] fp32, out [T, W] fp32) with x = hist[n - 1]: the same pass also
    forms out = sum_{j < n} coef[j] hist[j] (`depth_mix` with the updated x as the last term), and what is returned is
    `out` in the weight's dtype instead of x."""
    T, W = x.shape
    assert x.dtype == torch.float32 and W % groups == 0
    if history is not None:
        hist, n, coef, mix_out = history
        assert x.data_ptr() == hist[n - 1].data_ptr() and hist.is_contiguous() and mix_out.is_contiguous()
    if use_native(x):
        assert x.is_contiguous() and y.stride(1) == 1 and y.dtype in (weight.dtype, torch.float32)
        h = torch.empty(T, W, dtype=weight.dtype, device=x.device) if want_cast else None
        hargs = (None, _i64(0), 0, None, None) if history is None else \
            (loader.ptr(hist), _i64(hist.stride(0)), int(n), loader.ptr(coef), loader.ptr(mix_out))
        loader.check(_get_lib().cb_rmsnorm_residual(
            loader.ptr(x), loader.ptr(y), _i64(y.stride(0)), int(y.dtype == torch.float32 and weight.dtype != torch.float32),
            loader.ptr(weight), loader.ptr(h), _i64(T), W, int(groups), _f(eps), _f(mult), _f(offset), *hargs,
            code(weight.dtype), loader.stream_ptr()), "rmsnorm_residual")
        loader.launch_counter.add("rmsnorm_residual")
        return h
    x += mult * (_group_rms(y.float(), groups, eps) * (offset + weight.float()))
    if history is not None:
        return depth_mix(hist, n, coef, mix_out, cast_dtype=weight.dtype if want_cast else None)
    return x.to(weight.dtype) if want_cast else None


def rms_norm_f32in(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float = 0.0, groups: int = 1) -> torch.Tensor:
    """x [T, W] fp32 (unit stride inside a row) -> x / rms(x) * (offset + weight) in the weight's dtype; with `groups` > 1
    every one of that many equal consecutive parts of the row is divided by its own root mean square."""
    T, W = x.shape
    assert W % groups == 0
    if use_native(x):
        assert x.stride(1) == 1 and x.dtype == torch.float32
        out = torch.empty(T, W, dtype=weight.dtype, device=x.device)
        loader.check(_get_lib().cb_rmsnorm_f32in(loader.ptr(x), _i64(x.stride(0)), loader.ptr(weight), loader.ptr(out),
                                                 _i64(T), W, int(groups), _f(eps), _f(offset), code(weight.dtype),
                                                 loader.stream_ptr()), "rmsnorm_f32in")
        loader.launch_counter.add("rmsnorm_f32in")
        return out
    return (_group_rms(x.float(), groups, eps) * (offset + weight.float())).to(weight.dtype)


def depth_mix(hist: torch.Tensor, n: int, coef: torch.Tensor, out: torch.Tensor,
              cast_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """Weighted sum over the history of an fp32 residual stream: out = sum_{j < n} coef[j] * hist[j], j ascending, in fp32.
    hist [slices, T, W] fp32 (contiguous), coef [>= n] fp32 on the device, out [T, W] fp32 (may be a later slice of
    `hist`).  With `cast_dtype` the sum is also returned in that dtype (what the next layer's GEMMs read)."""
    T, W = out.shape
    assert hist.dtype == torch.float32 and out.dtype == torch.float32 and coef.dtype == torch.float32 and n <= hist.shape[0]
    want = cast_dtype is not None and cast_dtype != torch.float32
    if use_native(hist) and (T * W) % 4 == 0:
        assert hist.is_contiguous() and out.is_contiguous() and coef.is_contiguous()
        h = torch.empty(T, W, dtype=cast_dtype, device=out.device) if want else None
        loader.check(_get_lib().cb_depth_mix(loader.ptr(hist), _i64(hist.stride(0)), int(n), loader.ptr(coef),
                                             loader.ptr(out), loader.ptr(h), _i64(T * W),
                                             code(cast_dtype if want else torch.float32), loader.stream_ptr()), "depth_mix")
        loader.launch_counter.add("depth_mix")
        return h if want else (out if cast_dtype is not None else None)
    acc = coef[0] * hist[0]
    for j in range(1, n):
        acc = acc + coef[j] * hist[j]
    out.copy_(acc)
    return None if cast_dtype is None else out.to(cast_dtype)


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """z [T, F] -> a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(u) = u / sqrt(mean(u^2) + eps) over the
    row; coef = (a, b, c, e) fp32 on the device.  fp32 arithmetic, result in z's dtype."""
    T, Fw = z.shape
    if use_native(z):
        assert z.stride(1) == 1 and coef.dtype == torch.float32 and coef.numel() == 4 and coef.is_contiguous()
        out = torch.empty(T, Fw, dtype=z.dtype, device=z.device)
        loader.check(_get_lib().cb_poly_norm(loader.ptr(z), _i64(z.stride(0)), loader.ptr(out), _i64(T), Fw, loader.ptr(coef),
                                             _f(eps), code(z.dtype), loader.stream_ptr()), "poly_norm")
        loader.launch_counter.add("poly_norm")
        return out
    zf = z.float()
    c = coef.float()
    n = lambda u: u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)
    return (c[0] * n(zf) + c[1] * n(zf * zf) + c[2] * n(zf * zf * zf) + c[3]).to(z.dtype)


def head_rms_norm(x: torch.Tensor, heads_a: int, heads_b: int, dim: int, weight_a: torch.Tensor,
                  weight_b: Optional[torch.Tensor], eps: float, pages: Optional[tuple] = None) -> torch.Tensor:
    """x [T, >= (heads_a + heads_b) x dim] (unit stride inside a row): every head is divided by its root mean square over
    its `dim` channels and multiplied by a weight [dim] that the heads share - `weight_a` for the first `heads_a` heads
    (queries), `weight_b` for the next `heads_b` (keys).  Returns a new [T, (heads_a + heads_b) x dim] tensor.

    `pages` = (k_cache, v_cache [blocks, block_size, heads_b, dim], block_tables, meta): the normed key heads are written
    into the tokens' rows of `k_cache` and the key heads AS THEY CAME IN into `v_cache` (attention whose values are its keys
    before their norm); only the query heads [T, heads_a x dim] are returned."""
    T = x.shape[0]
    H = heads_a + heads_b
    if pages is not None:
        k_cache, v_cache, block_tables, meta = pages
        bs = k_cache.shape[1]
        assert k_cache.shape[2:] == (heads_b, dim) and v_cache.shape == k_cache.shape and k_cache.dtype == x.dtype
    if use_native(x):
        assert x.stride(1) == 1 and weight_a.dtype == x.dtype and (weight_b is None or weight_b.dtype == x.dtype)
        out = torch.empty(T, (heads_a if pages is not None else H) * dim, dtype=x.dtype, device=x.device)
        pargs = (None, None, None, None, None, 0, 0) if pages is None else \
            (loader.ptr(k_cache), loader.ptr(v_cache), loader.ptr(block_tables), loader.ptr(meta.token_seq),
             loader.ptr(meta.token_pos), bs, block_tables.shape[1])
        if pages is not None:
            assert k_cache.is_contiguous() and v_cache.is_contiguous() and v_cache.dtype == x.dtype
        loader.check(_get_lib().cb_head_rmsnorm(loader.ptr(x), _i64(x.stride(0)), loader.ptr(out), _i64(out.stride(0)),
                                                _i64(T), H, heads_a, dim, loader.ptr(weight_a), loader.ptr(weight_b), _f(eps),
                                                *pargs, code(x.dtype), loader.stream_ptr()), "head_rmsnorm")
        loader.launch_counter.add("head_rmsnorm")
        return out
    y = x[:, : H * dim].float().reshape(T, H, dim)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    w = torch.cat([weight_a.float()[None].expand(heads_a, dim)] +
                  ([weight_b.float()[None].expand(heads_b, dim)] if heads_b else []), 0)
    y = (y * w[None]).reshape(T, H * dim).to(x.dtype)
    if pages is None:
        return y
    blk = block_tables[meta.token_seq.long(), (meta.token_pos // bs).long()].long()
    off = (meta.token_pos % bs).long()
    k_cache.view(k_cache.shape[0], bs, heads_b * dim)[blk, off] = y[:, heads_a * dim:]
    v_cache.view(v_cache.shape[0], bs, heads_b * dim)[blk, off] = x[:, heads_a * dim: H * dim]
    return y[:, : heads_a * dim].contiguous()


def norm_mean(parts: Sequence[torch.Tensor], weights: Sequence[torch.Tensor], eps: float) -> torch.Tensor:
    """Mean of RMS-normed tensors: (1 / n) sum_i parts[i] / sqrt(mean(parts[i]^2) + eps) * weights[i], every part
    [T, W] (compute dtype or fp32, unit stride inside a row) normalised over W in fp32.  Returns fp32 [T, W]: the
    output of mixers that run side by side, ready to be added to an fp32 residual stream."""
    n = len(parts)
    T, W = parts[0].shape
    assert 1 <= n <= 4 and len(weights) == n
    if use_native(parts[0]):
        out = torch.empty(T, W, dtype=torch.float32, device=parts[0].device)
        ps = list(parts) + [None] * (4 - n)
        ws = list(weights) + [None] * (4 - n)
        assert all(p.stride(1) == 1 and p.shape == (T, W) for p in parts)
        assert all(w.is_contiguous() and w.dtype == p.dtype for w, p in zip(weights, parts))
        args = []
        for p_, w_ in zip(ps, ws):
            args += [loader.ptr(p_), _i64(0 if p_ is None else p_.stride(0)), loader.ptr(w_),
                     code(p_.dtype) if p_ is not None else 0]
        loader.check(_get_lib().cb_norm_mean(*args, n, loader.ptr(out), _i64(T), W, _f(eps), loader.stream_ptr()),
                     "norm_mean")
        loader.launch_counter.add("norm_mean")
        return out
    acc = None
    for p_, w_ in zip(parts, weights):
        pf = p_.float()
        y = pf / torch.sqrt((pf * pf).mean(-1, keepdim=True) + eps) * w_.float()
        acc = y if acc is None else acc + y
    return acc * (1.0 / n)


def sigmoid_gate_mul(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """o [T, C] (contiguous) times sigmoid(gate [T, C], unit stride inside a row), in place; the sigmoid in fp32."""
    T, C = o.shape
    if use_native(o):
        assert o.is_contiguous() and gate.stride(1) == 1 and gate.dtype == o.dtype and gate.shape == o.shape
        loader.check(_get_lib().cb_sigmoid_gate_mul(loader.ptr(o), loader.ptr(gate), _i64(gate.stride(0)), _i64(T), C,
                                                    code(o.dtype), loader.stream_ptr()), "sigmoid_gate_mul")
        loader.launch_counter.add("sigmoid_gate_mul")
        return o
    o.copy_((o.float() * torch.sigmoid(gate.float())).to(o.dtype))
    return o


def rotary_unit_norm(x: torch.Tensor, heads: int, dim: int, rot_dims: int, interleaved: bool,
                     table: Optional[torch.Tensor], token_pos: torch.Tensor, unit_eps: Optional[float]) -> None:
    """In place on the first `heads x dim` columns of x [T, .]: every head's first `rot_dims` channels are turned by the
    token's position - pairs (2i, 2i + 1) when `interleaved`, else (i, i + rot_dims / 2); `table` = `rotary_table` of
    `rot_dims` - and then, with `unit_eps`, the head is divided by sqrt(mean of its squares + unit_eps).  fp32
    arithmetic, one rounding into x's dtype."""
    T = x.shape[0]
    if rot_dims == 0 and unit_eps is None:
        return
    if use_native(x):
        assert x.stride(1) == 1 and (rot_dims == 0 or (table.dtype == torch.float32 and table.shape[1] == rot_dims))
        loader.check(_get_lib().cb_rotary_unit_norm(
            loader.ptr(x), _i64(x.stride(0)), _i64(T), heads, dim, rot_dims, int(interleaved),
            loader.ptr(table if rot_dims else None), loader.ptr(token_pos), int(unit_eps is not None),
            _f(unit_eps or 0.0), code(x.dtype), loader.stream_ptr()), "rotary_unit_norm")
        loader.launch_counter.add("rotary_unit_norm")
        return
    y = x[:, : heads * dim].float().reshape(T, heads, dim)
    if rot_dims:
        half = rot_dims // 2
        cs = table[token_pos.long()]
        c, sn = cs[:, None, :half], cs[:, None, half:]
        if interleaved:
            a, b = y[..., 0:rot_dims:2], y[..., 1:rot_dims:2]
            rot = torch.stack([a * c - b * sn, b * c + a * sn], -1).reshape(T, heads, rot_dims)
        else:
            a, b = y[..., :half], y[..., half:rot_dims]
            rot = torch.cat([a * c - b * sn, b * c + a * sn], -1)
        y = torch.cat([rot, y[..., rot_dims:]], -1)
    if unit_eps is not None:
        y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + unit_eps)
    x[:, : heads * dim] = y.reshape(T, heads * dim).to(x.dtype)


_NORM_KINDS = {None: 0, "none": 0, "rms": 1, "layer": 2}


def stream_add_norm(x: torch.Tensor, addends: Sequence[torch.Tensor] = (), row: Optional[torch.Tensor] = None,
                    weight: Optional[torch.Tensor] = None, eps: float = 1e-5, kind: Optional[str] = None,
                    offset: float = 0.0, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """The fp32 residual stream x [T, W], updated in place: x += sum(addends) (+ `row` [W] for every token), the addends
    summed among themselves first, all in fp32.  Addends are [T, W] in the compute dtype or fp32 (at most four).  With
    `kind` "rms" / "layer" the new x is normalised in the same pass - x / sqrt(mean x^2 + eps) or
    (x - mean) / sqrt(mean of squared deviations + eps), times (offset + weight) - and returned in `out_dtype` (default: the
    weight's dtype).  One kernel sums a layer's sublayer outputs into the stream and feeds the next layer's GEMMs."""
    T, W = x.shape
    assert x.dtype == torch.float32 and len(addends) <= 4
    k = _NORM_KINDS[kind]
    if k and out_dtype is None:
        out_dtype = weight.dtype
    if use_native(x):
        assert x.is_contiguous() and all(a.stride(1) == 1 and a.shape == x.shape for a in addends)
        h = torch.empty(T, W, dtype=out_dtype, device=x.device) if k else None
        if row is not None:
            row = row.float().contiguous()
        ad = list(addends) + [None] * (4 - len(addends))
        loader.check(_get_lib().cb_stream_add_norm(
            loader.ptr(x), loader.ptr(ad[0]), _i64(0 if ad[0] is None else ad[0].stride(0)),
            code(ad[0].dtype) if ad[0] is not None else 0, loader.ptr(ad[1]), _i64(0 if ad[1] is None else ad[1].stride(0)),
            code(ad[1].dtype) if ad[1] is not None else 0, loader.ptr(ad[2]), _i64(0 if ad[2] is None else ad[2].stride(0)),
            code(ad[2].dtype) if ad[2] is not None else 0, loader.ptr(ad[3]), _i64(0 if ad[3] is None else ad[3].stride(0)),
            code(ad[3].dtype) if ad[3] is not None else 0, loader.ptr(row),
            loader.ptr(weight if k else None), code(weight.dtype) if (k and weight is not None) else 0, loader.ptr(h),
            code(out_dtype) if k else 0, _i64(T), W, k, _f(eps), _f(offset), loader.stream_ptr()), "stream_add_norm")
        loader.launch_counter.add("stream_add_norm")
        return h
    if len(addends) or row is not None:
        acc = None
        for a in addends:
            acc = a.float() if acc is None else acc + a.float()
        if row is not None:
            acc = row.float()[None, :] if acc is None else acc + row.float()[None, :]
        x += acc
    if not k:
        return None
    if k == 1:
        y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    else:
        d = x - x.mean(-1, keepdim=True)
        y = d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps)
    return (y * (offset + weight.float())).to(out_dtype)


# ------------------------------------------------------------------------------------------------ paged attention
def latent_kv_write(z: torch.Tensor, norm_weight: torch.Tensor, eps: float, kv_rank: int, rot_table: torch.Tensor,
                    cache: torch.Tensor, block_tables: torch.Tensor, meta: RaggedMeta) -> None:
    """The cache rows of latent attention.  z [T, kv_rank + rot]: the first `kv_rank` columns are RMS-normalised with
    `norm_weight` (the latent), the others are turned by the token's position (the rotated key part all heads share);
    both go, rounded once, into the token's row of the paged cache [blocks, block_size, 1, kv_rank + rot]."""
    T, Wz = z.shape
    rot = Wz - kv_rank
    bs = cache.shape[1]
    if use_native(z):
        assert z.stride(1) == 1 and cache.is_contiguous() and cache.shape[-1] == Wz and rot_table.shape[1] == rot
        loader.check(_get_lib().cb_latent_kv_write(
            loader.ptr(z), _i64(z.stride(0)), loader.ptr(norm_weight), code(norm_weight.dtype), _f(eps), kv_rank, rot,
            loader.ptr(rot_table), loader.ptr(cache), loader.ptr(block_tables), loader.ptr(meta.token_seq),
            loader.ptr(meta.token_pos), _i64(T), bs, block_tables.shape[1], code(z.dtype), loader.stream_ptr()),
            "latent_kv_write")
        loader.launch_counter.add("latent_kv_write")
        return
    zf = z.float()
    c = zf[:, :kv_rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * norm_weight.float()
    kr = _rot_ref(zf[:, None, kv_rank:], meta.token_pos, rot_table, rot)[:, 0]
    blk = block_tables[meta.token_seq.long(), (meta.token_pos // bs).long()].long()
    off = (meta.token_pos % bs).long()
    cache.view(cache.shape[0], bs, Wz)[blk, off] = torch.cat([c, kr], -1).to(cache.dtype)


def paged_kv_write_mix(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                       block_tables: torch.Tensor, meta: RaggedMeta, v_other: Optional[torch.Tensor] = None,
                       lam: float = 0.0) -> None:
    """k [T, Gk x dim], v [T, Gv x vdim] rows into caches [blocks, block_size, G, dim] / [.., G, vdim]; with `v_other`
    the stored values are (1 - lam) v + lam v_other."""
    T = k.shape[0]
    bs = k_cache.shape[1]
    kw, vw = k.shape[1], v.shape[1]
    if use_native(k):
        assert k.stride(1) == 1 and v.stride(1) == 1 and k_cache.dtype == k.dtype and v_cache.dtype == v.dtype
        loader.check(_get_lib().cb_paged_kv_write_mix(
            loader.ptr(k), _i64(k.stride(0)), loader.ptr(v), _i64(v.stride(0)), loader.ptr(v_other),
            _i64(0 if v_other is None else v_other.stride(0)), _f(lam), loader.ptr(k_cache), loader.ptr(v_cache),
            loader.ptr(block_tables), loader.ptr(meta.token_seq), loader.ptr(meta.token_pos), _i64(T), kw, vw, bs,
            block_tables.shape[1], code(k.dtype), loader.stream_ptr()), "paged_kv_write_mix")
        loader.launch_counter.add("paged_kv_write_mix")
        return
    if v_other is not None:
        v = ((1.0 - lam) * v.float() + lam * v_other.float()).to(v.dtype)
    blk = block_tables[meta.token_seq.long(), (meta.token_pos // bs).long()].long()
    off = (meta.token_pos % bs).long()
    k_cache.view(k_cache.shape[0], bs, kw)[blk, off] = k
    v_cache.view(v_cache.shape[0], bs, vw)[blk, off] = v


def paged_bias_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                         meta: RaggedMeta, scale: float, bias_table: Optional[torch.Tensor] = None,
                         bucket_starts: Optional[torch.Tensor] = None, sink: bool = False,
                         lut: Optional[torch.Tensor] = None, tensor_cores: Optional[bool] = None,
                         vdim: Optional[int] = None, mask_block: int = 0, wide_weights: bool = False,
                         sink_values: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
                         window: int = 0) -> torch.Tensor:
    """Causal attention of every step token over positions 0..pos of its sequence in the paged cache; with `mask_block`
    only over the positions of its own block, floor(pos / mask_block) * mask_block .. pos (blocks are counted from the
    start of the sequence, whatever the step's cut).
    With `vdim` given and `v_cache` the key cache itself, the values are the first `vdim` columns of the key rows (latent
    attention: one row per token serves as key and value).
    q [T, heads x dim]; caches [blocks, block_size, kv_heads, dim | vdim]; bias_table [buckets, heads] fp32 indexed by
    the bucket of the distance (`bucket_starts` [buckets] int32: smallest distance of each bucket); `sink` adds a key of
    score 0 without a value to the softmax - with `sink_values` [heads] fp32 a key of that (unscaled) score per head.
    `slopes` [heads] fp32 takes slope * (pos - key position) off every score; `window` > 0 keeps only the keys
    pos - window + 1 .. pos.  Returns [T, heads x vdim].

    Two kernels: 16-bit inputs whose head widths are multiples of 8 up to 256 run on tensor cores (`lut` = `bucket_lut`
    of the same buckets; built here when absent); everything else - fp32 above all - takes the exact CUDA-core kernel.
    `tensor_cores` forces the choice.  `wide_weights`: the tensor-core kernel feeds the softmax weights into the
    weighted sum of the values as two 16-bit terms (value + rest of its rounding) instead of one, which keeps about 16
    bits of every weight; the exact kernel holds them in fp32 anyway."""
    T = q.shape[0]
    _, bs, G, dim = k_cache.shape
    ldv = v_cache.shape[3]                     # elements between the value rows of consecutive (token, kv head) pairs
    vdim = ldv if vdim is None else vdim
    heads = q.shape[1] // dim
    nb = 0 if bias_table is None else bias_table.shape[0]
    if use_native(q):
        if vdim > 512:
            raise NotImplementedError("paged_bias_attention: value width above 512 is not supported")
        assert q.stride(1) == 1 and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype
        out = torch.empty(T, heads * vdim, dtype=q.dtype, device=q.device)
        mma_ok = (q.dtype in (torch.bfloat16, torch.float16) and dim % 8 == 0 and vdim % 8 == 0 and dim <= 256
                  and vdim <= 256 and nb <= 255 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and ldv % 8 == 0)
        if tensor_cores is None:
            tensor_cores = mma_ok
        if tensor_cores:
            if not mma_ok:
                raise ValueError("paged_bias_attention: the tensor-core kernel needs 16-bit inputs and head widths "
                                 "that are multiples of 8 up to 256")
            if nb and lut is None:
                lut = bucket_lut(bucket_starts.tolist()).to(q.device)
            # few CTAs (decode steps): split the keys so that about two waves of CTAs run, join the parts afterwards
            R = heads // G
            tiles = meta.nseq * G * ((meta.max_q * R + 63) // 64)
            max_len = max(c + n for c, n in zip(meta.ctx_lens, meta.q_lens))
            if mask_block:
                max_len = min(max_len, mask_block + 64)       # keys a tile can see: the split is sized for those
            if window:
                max_len = min(max_len, window + 64)
            chunk = splits = 0
            part_o = part_ml = None
            if tiles < _SPLIT_BELOW_TILES and max_len >= 256:
                chunk = max(128, -(-(max_len * tiles // (2 * _SPLIT_BELOW_TILES)) // 64) * 64)
                splits = -(-max_len // chunk)
                if splits > 1:
                    part_o = _workspace("attn_o", T * heads * splits * vdim, q.device)
                    part_ml = _workspace("attn_ml", T * heads * splits * 2, q.device)
                else:
                    chunk = splits = 0
            if (mask_block or window) and splits:
                max_len = max(c + n for c, n in zip(meta.ctx_lens, meta.q_lens))
                splits = -(-max_len // chunk)                 # chunks are counted from key 0
                part_o = _workspace("attn_o", T * heads * splits * vdim, q.device)
                part_ml = _workspace("attn_ml", T * heads * splits * 2, q.device)
            loader.check(_get_lib().cb_paged_bias_attention_mma(
                loader.ptr(q), _i64(q.stride(0)), loader.ptr(k_cache), loader.ptr(v_cache), loader.ptr(block_tables),
                loader.ptr(meta.cu_q), loader.ptr(meta.ctx_len), loader.ptr(meta.token_pos), loader.ptr(bias_table),
                loader.ptr(lut), 0 if lut is None else lut.numel(), nb, loader.ptr(out), _i64(T), meta.nseq, meta.max_q,
                heads, G, dim, vdim, ldv, bs, block_tables.shape[1], _f(scale), int(sink), chunk, splits,
                loader.ptr(part_o), loader.ptr(part_ml), int(mask_block), int(wide_weights), loader.ptr(sink_values),
                loader.ptr(slopes), int(window), code(q.dtype), loader.stream_ptr()),
                "paged_bias_attention_mma")
            loader.launch_counter.add("paged_bias_attention_mma")
            return out
        loader.check(_get_lib().cb_paged_bias_attention(
            loader.ptr(q), _i64(q.stride(0)), loader.ptr(k_cache), loader.ptr(v_cache), loader.ptr(block_tables),
            loader.ptr(meta.token_seq), loader.ptr(meta.token_pos), loader.ptr(bias_table), loader.ptr(bucket_starts), nb,
            loader.ptr(out), _i64(T), heads, G, dim, vdim, ldv, bs, block_tables.shape[1], _f(scale), int(sink),
            int(mask_block), loader.ptr(sink_values), loader.ptr(slopes), int(window), code(q.dtype),
            loader.stream_ptr()), "paged_bias_attention")
        loader.launch_counter.add("paged_bias_attention")
        return out
    out = torch.empty(T, heads * vdim, dtype=q.dtype)
    rep = heads // G
    t0 = 0
    for i, (n, c) in enumerate(zip(meta.q_lens, meta.ctx_lens)):
        if n == 0:
            continue
        L = c + n
        blks = block_tables[i, :(L + bs - 1) // bs].long()
        kk = k_cache[blks].reshape(-1, G, dim)[:L].float().repeat_interleave(rep, 1)
        vv = v_cache[blks].reshape(-1, G, ldv)[:L, :, :vdim].float().repeat_interleave(rep, 1)
        qq = q[t0:t0 + n].float().view(n, heads, dim)
        s = torch.einsum("ihd,jhd->hij", qq, kk) * scale
        dist = torch.arange(c, L)[:, None] - torch.arange(L)[None, :]
        if bias_table is not None:
            b = torch.bucketize(dist.clamp(min=0), bucket_starts.to(torch.int64), right=True) - 1
            s = s + bias_table.float()[b].permute(2, 0, 1)
        s = s.masked_fill(dist[None] < 0, float("-inf"))
        if mask_block:
            same = (torch.arange(c, L)[:, None] // mask_block) == (torch.arange(L)[None, :] // mask_block)
            s = s.masked_fill(~same[None], float("-inf"))
        if window:
            s = s.masked_fill(dist[None] >= window, float("-inf"))
        if slopes is not None:
            s = s - slopes.float()[:, None, None] * dist.clamp(min=0)[None].float()
        if sink:
            sv = torch.zeros(heads) if sink_values is None else sink_values.float()
            s = torch.cat([s, sv[:, None, None].expand(heads, n, 1)], -1)
        p = torch.softmax(s, -1)[..., :L]
        out[t0:t0 + n] = torch.einsum("hij,jhv->ihv", p, vv).reshape(n, heads * vdim).to(q.dtype)
        t0 += n
    return out
