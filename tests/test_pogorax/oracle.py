"""Plain, slow float64 implementation of the Pogorax decoder, one function per mechanism, written from the equations and
sharing no code with the package: the yardstick for the kernels, the ragged step function and the engine.

Notation: h is a sublayer's normalised input [L, width]; all products are W h with W stored [out, in]; positions count
from 0.  A layer is x <- x + mixer(rms(x) w1), then (where it has a feed-forward) x <- x + ff(rms(x) w2).  Every
recurrence walks the tokens one by one from a zero state.
"""
import json
import math
import os

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------------------------- small pieces
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + x.clamp(min=0)


def log_sigmoid(x):
    return -softplus(-x)


def rotate_pairs(x, pos, dims, base):
    """x [L, H, d]; channels 2i and 2i + 1 (i < dims / 2) of every head turn by the angle pos * base^(-2i/dims); the
    other channels pass."""
    out = x.clone()
    for t in range(x.shape[0]):
        for i in range(dims // 2):
            a = float(pos[t]) * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = u * c - v * s
            out[t, :, 2 * i + 1] = v * c + u * s
    return out


def short_conv(x, w, b):
    """Causal convolution per channel: x [L, C], w [C, taps] with the last column on the current token, zeros before the
    first token; b [C] is added."""
    L, C = x.shape
    taps = w.shape[1]
    out = torch.zeros(L, C, dtype=x.dtype)
    for t in range(L):
        for i in range(taps):
            src = t - (taps - 1) + i
            if src >= 0:
                out[t] += w[:, i] * x[src]
    return out + b


# ----------------------------------------------------------------------------------------------- mixers
def softmax_attention(h, W, p, mx, eps, pos, unit_norm, gated):
    """Grouped-query softmax attention.  Options: rotary pairs on the first channels of q / k heads (`rot`), q and k
    brought to unit RMS per head afterwards, a block mask (`mask.size`: only keys of the query's own block of positions,
    counted from position 0), a sigmoid gate on the heads' outputs."""
    L = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ W[p + "q"].T).view(L, H, d)
    k = (h @ W[p + "k"].T).view(L, G, d)
    v = (h @ W[p + "v"].T).view(L, G, dv)
    if mx.get("rot"):
        q = rotate_pairs(q, pos, mx["rot"]["dims"], mx["rot"]["base"])
        k = rotate_pairs(k, pos, mx["rot"]["dims"], mx["rot"]["base"])
    if unit_norm:
        q, k = rms(q, eps), rms(k, eps)
    size = (mx.get("mask") or {}).get("size")
    out = torch.zeros(L, H, dv, dtype=h.dtype)
    for n in range(H):
        g = n // (H // G)
        for i in range(L):
            first = (pos[i] // size) * size if size else 0
            js = [j for j in range(L) if first <= pos[j] <= pos[i]]
            s = (k[js, g] @ q[i, n]) * mx["scale"]
            out[i, n] = torch.softmax(s, 0) @ v[js, g]
    o = out.reshape(L, H * dv)
    if gated:
        o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def matrix_memory(h, W, p, mx, eps):
    """Per head a matrix S [d, dv], a vector n [d] and a running maximum m, all zero at the start.  Log gates
    i = cap tanh(. / cap), f = log sigmoid(cap tanh(. / cap)); m' = max(f + m, i); S and n are scaled by exp(f + m - m') and
    take exp(i - m') k v^T resp. exp(i - m') k; the read-out S^T q / (max(|n . q|, exp(-m')) + 1e-6) with q scaled by d^-1/2
    is brought to unit RMS per head, weighted, gated by a sigmoid and projected."""
    L = h.shape[0]
    H, d, dv, cap = mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    q = (h @ W[p + "q"].T).view(L, H, d) * d ** -0.5
    k = (h @ W[p + "k"].T).view(L, H, d)
    v = (h @ W[p + "v"].T).view(L, H, dv)
    ig = cap * torch.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    fg = log_sigmoid(cap * torch.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    out = torch.zeros(L, H, dv, dtype=h.dtype)
    for n_ in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        nv = torch.zeros(d, dtype=h.dtype)
        m = torch.zeros((), dtype=h.dtype)
        for t in range(L):
            m_new = torch.maximum(fg[t, n_] + m, ig[t, n_])
            keep, take = torch.exp(fg[t, n_] + m - m_new), torch.exp(ig[t, n_] - m_new)
            S = keep * S + take * torch.outer(k[t, n_], v[t, n_])
            nv = keep * nv + take * k[t, n_]
            m = m_new
            den = torch.maximum((nv @ q[t, n_]).abs(), torch.exp(-m)) + 1e-6
            out[t, n_] = (S.T @ q[t, n_]) / den
    o = rms(out, eps).reshape(L, H * dv) * W[p + "norm"]
    o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def linear_recurrent_unit(h, W, p, mx):
    """Two branches: y = gelu_tanh(W_y h + b) and u = conv(W_x h + b).  Per block of channels r = sigmoid(A u + a),
    i = sigmoid(I u + i0); decay = exp(-8 r softplus(lam)); S <- decay S + sqrt(1 - decay^2) i u per channel; output
    W_o (S y)."""
    L = h.shape[0]
    C, nb = mx["width"], mx["blocks"]
    bw = C // nb
    y = gelu_tanh(h @ W[p + "y"].T + W[p + "y.b"])
    u = short_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    r = torch.zeros(L, C, dtype=h.dtype)
    ig = torch.zeros(L, C, dtype=h.dtype)
    for b in range(nb):
        ub = u[:, b * bw:(b + 1) * bw]
        r[:, b * bw:(b + 1) * bw] = torch.sigmoid(ub @ W[p + "ra"][b].T + W[p + "ra.b"][b])
        ig[:, b * bw:(b + 1) * bw] = torch.sigmoid(ub @ W[p + "ri"][b].T + W[p + "ri.b"][b])
    decay = torch.exp(-8.0 * r * softplus(W[p + "lam"]))
    S = torch.zeros(C, dtype=h.dtype)
    out = torch.zeros(L, C, dtype=h.dtype)
    for t in range(L):
        S = decay[t] * S + torch.sqrt(1.0 - decay[t] ** 2) * ig[t] * u[t]
        out[t] = S
    return (out * y) @ W[p + "o"].T


def state_space(h, W, p, mx, eps):
    """W_in h = [z | x | B | C | dt]; x | B | C through a causal convolution and silu; step = softplus(dt + bias); per head
    S <- exp(-exp(A_log) step) S + step B x^T, y = S^T C + D x; y silu(z) is RMS-normed in equal parts, weighted, projected."""
    L = h.shape[0]
    H, dv, N, G, parts = mx["heads"], mx["vdim"], mx["state"], mx["groups"], mx["norm_groups"]
    inner = H * dv
    zz = h @ W[p + "in"].T
    z, xbc, dt = zz[:, :inner], zz[:, inner:2 * inner + 2 * G * N], zz[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(L, H, dv)
    B = xbc[:, inner:inner + G * N].view(L, G, N)
    C = xbc[:, inner + G * N:].view(L, G, N)
    step = softplus(dt + W[p + "dt_bias"])
    y = torch.zeros(L, H, dv, dtype=h.dtype)
    for n in range(H):
        g = n // (H // G)
        S = torch.zeros(N, dv, dtype=h.dtype)
        for t in range(L):
            S = torch.exp(-torch.exp(W[p + "A_log"][n]) * step[t, n]) * S + step[t, n] * torch.outer(B[t, g], x[t, n])
            y[t, n] = S.T @ C[t, g] + W[p + "D"][n] * x[t, n]
    y = y.reshape(L, inner) * silu(z)
    y = rms(y.view(L, parts, inner // parts), eps).reshape(L, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def pair(h, W, p, ly, eps, pos):
    """Two mixers on the same input; each output is RMS-normed over the width with its own weight; half their sum."""
    mx = ly["mixer"]
    if ly["type"] == "parallel":
        a = softmax_attention(h, W, p + "left.", mx["left"], eps, pos, unit_norm=False, gated=True)
        b = matrix_memory(h, W, p + "right.", mx["right"], eps)
    else:
        a = softmax_attention(h, W, p + "left.", mx["left"], eps, pos, unit_norm=True, gated=False)
        b = linear_recurrent_unit(h, W, p + "right.", mx["right"])
    return 0.5 * (rms(a, eps) * W[p + "left.out"] + rms(b, eps) * W[p + "right.out"])


def gated_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# ----------------------------------------------------------------------------------------------- the model
def forward(cfg, W, tokens, layers_out=None):
    """Logits [L, vocab] of one sequence; `layers_out` (a list) receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    L = len(tokens)
    pos = list(range(L))
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, ly in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * W[p + "norm1"]
        if ly["type"] == "mamba2":
            x = x + state_space(h, W, p + "mix.", ly["mixer"], eps)
        else:
            x = x + pair(h, W, p + "mix.", ly, eps, pos)
        if ly["mlp"] is not None:
            x = x + gated_ff(rms(x, eps) * W[p + "norm2"], W, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T


# ----------------------------------------------------------------------------------------------- test models
def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def _mlp(mlp):
    return dense() if mlp == "dense" else mlp


def gated_pair_layer(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, mask=12, m_heads=3, m_dim=8, m_vdim=16, cap=6.0,
                     mlp="dense"):
    """Block-masked gated attention beside the matrix memory."""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if mask:
        left["mask"] = {"size": mask}
    return {"type": "parallel", "mlp": _mlp(mlp),
            "mixer": {"left": left, "right": {"heads": m_heads, "dim": m_dim, "vdim": m_vdim, "gate_cap": cap}}}


def rotary_pair_layer(heads=4, kv_heads=1, dim=16, vdim=16, scale=0.25, rot_dims=8, base=1000.0, width=32, blocks=2,
                      conv=4, mlp="dense"):
    """Rotary unit-norm attention beside the linear recurrent unit."""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        left["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "parallel_2", "mlp": _mlp(mlp),
            "mixer": {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv}}}


def state_space_layer(heads=4, vdim=8, state=16, groups=2, norm_groups=2, conv=4, mlp=None):
    return {"type": "mamba2", "mlp": _mlp(mlp),
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups,
                      "conv": conv}}


def make_config(layers, width=48, vocab=96, eps=1e-5, embed_scale=3.0):
    return {"architecture": "Pogorax", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def random_weights(cfg, seed=0):
    """name -> bf16-representable fp32 tensors in the checkpoint's naming."""
    gen = torch.Generator().manual_seed(seed)
    W, Wd = {}, cfg["width"]

    def lin(o, i, s=1.0):
        return torch.randn(o, i, generator=gen) * (s / math.sqrt(i))

    def vec(n, mean=0.0, std=0.2):
        return mean + torch.randn(n, generator=gen) * std

    W["embed"] = torch.randn(cfg["vocab"], Wd, generator=gen) * 0.5
    W["head"] = lin(cfg["vocab"], Wd)
    W["final.norm"] = vec(Wd, 1.0)
    for i, ly in enumerate(cfg["layers"]):
        p, mx, mlp = f"l{i}.", ly["mixer"], ly["mlp"]
        W[p + "norm1"] = vec(Wd, 1.0)
        if mlp is not None:
            W[p + "norm2"] = vec(Wd, 1.0)
            W[p + "mlp.gate"], W[p + "mlp.up"] = lin(mlp["ff"], Wd, 1.5), lin(mlp["ff"], Wd, 1.5)
            W[p + "mlp.down"] = lin(Wd, mlp["ff"])
        p += "mix."
        if ly["type"] == "mamba2":
            H, dv, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
            inner, ch = H * dv, H * dv + 2 * G * N
            W[p + "in"] = lin(inner + ch + H, Wd, 1.5)
            W[p + "conv"] = torch.randn(ch, mx["conv"], generator=gen) * 0.5
            W[p + "conv.b"] = vec(ch)
            W[p + "dt_bias"] = vec(H, -1.0, 1.0)
            W[p + "A_log"] = vec(H, -0.5, 1.0)
            W[p + "D"] = vec(H, 1.0, 0.5)
            W[p + "norm"] = vec(inner, 1.0)
            W[p + "o"] = lin(Wd, inner)
            continue
        lm, rm = mx["left"], mx["right"]
        H, G, d, dv = lm["heads"], lm["kv_heads"], lm["dim"], lm["vdim"]
        q = p + "left."
        W[q + "q"], W[q + "k"], W[q + "v"] = lin(H * d, Wd, 2.0), lin(G * d, Wd, 2.0), lin(G * dv, Wd)
        W[q + "o"] = lin(Wd, H * dv)
        W[q + "out"] = vec(Wd, 1.0)
        r = p + "right."
        W[r + "out"] = vec(Wd, 1.0)
        if ly["type"] == "parallel":
            W[q + "g"] = lin(H * dv, Wd, 2.0)
            Hm, dm, dvm = rm["heads"], rm["dim"], rm["vdim"]
            W[r + "q"], W[r + "k"], W[r + "v"] = lin(Hm * dm, Wd, 2.0), lin(Hm * dm, Wd, 2.0), lin(Hm * dvm, Wd)
            W[r + "g"] = lin(Hm * dvm, Wd, 2.0)
            W[r + "i"], W[r + "f"] = lin(Hm, Wd, 3.0), lin(Hm, Wd, 3.0)
            W[r + "i.b"], W[r + "f.b"] = vec(Hm, 0.0, 1.0), vec(Hm, 2.0, 1.0)
            W[r + "norm"] = vec(Hm * dvm, 1.0)
            W[r + "o"] = lin(Wd, Hm * dvm)
        else:
            C, nb = rm["width"], rm["blocks"]
            W[r + "y"], W[r + "x"] = lin(C, Wd, 1.5), lin(C, Wd, 1.5)
            W[r + "y.b"], W[r + "x.b"] = vec(C), vec(C)
            W[r + "conv"] = torch.randn(C, rm["conv"], generator=gen) * 0.5
            W[r + "conv.b"] = vec(C)
            W[r + "ra"] = torch.randn(nb, C // nb, C // nb, generator=gen) / math.sqrt(C // nb)
            W[r + "ri"] = torch.randn(nb, C // nb, C // nb, generator=gen) / math.sqrt(C // nb)
            W[r + "ra.b"], W[r + "ri.b"] = vec(C, 0.0, 1.0).view(nb, -1), vec(C, 0.0, 1.0).view(nb, -1)
            W[r + "lam"] = vec(C, -1.0, 1.5)
            W[r + "o"] = lin(Wd, C)
    return {k: v.to(torch.bfloat16).float() for k, v in W.items()}


def write_checkpoint(folder, cfg, W):
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in W.items()}, os.path.join(folder, "model.safetensors"))
    return str(folder)


def to64(W):
    return {k: v.to(F64) for k, v in W.items()}
