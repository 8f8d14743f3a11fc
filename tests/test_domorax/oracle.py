"""Plain, slow float64 implementation of the Domorax decoder, one function per mechanism, written from the equations and
sharing no code with the package: the yardstick for the kernels, the ragged step function and the engine.

Notation: h is a sublayer's input [L, width] (the residual stream itself: only sublayer OUTPUTS are normalised); all
products are W h with W stored [out, in]; positions count from 0.  A layer is x <- x + m gn(mixer(x)) w1, then (where it
has a feed-forward) x <- x + m gn(ff(x)) w2, with gn the RMS norm in equal consecutive groups.  What the next layer reads
is a learned weighted sum of the embedding output and of all layer results so far.
"""
import json
import math
import os

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------------------------- small pieces
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_rms(x, groups, eps):
    """RMS norm in `groups` equal consecutive parts of the last axis."""
    L, C = x.shape
    return rms(x.view(L, groups, C // groups), eps).reshape(L, C)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + x.clamp(min=0)


def short_conv(x, w):
    """Causal convolution per channel: x [L, C], w [C, taps] with the last column on the current token, zeros before the
    first token, no bias."""
    L, C = x.shape
    taps = w.shape[1]
    out = torch.zeros(L, C, dtype=x.dtype)
    for t in range(L):
        for i in range(taps):
            src = t - (taps - 1) + i
            if src >= 0:
                out[t] += w[:, i] * x[src]
    return out


def rotary_frequencies(rot):
    """f_i = base^(-2i/dims) for i < dims/2, and the factor on cos / sin.  With `scaling` (factor s, original length n,
    fast, slow): d(t) = dims ln(n / (2 pi t)) / (2 ln base); lo = max(floor(d(fast)), 0); hi = min(ceil(d(slow)), dims - 1);
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); f_i <- f_i / s r_i + f_i (1 - r_i); cos, sin times 0.1 ln s + 1."""
    dims, base = rot["dims"], float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    s, n = float(sc["factor"]), float(sc["original"])
    d = lambda t: dims * math.log(n / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(d(float(sc["fast"]))), 0)
    hi = min(math.ceil(d(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / s * r + fi * (1.0 - r))
    return out, 0.1 * math.log(s) + 1.0


def rotate_half(x, pos, rot):
    """x [L, H, d]: channel i < dims/2 of every head is paired with channel i + dims/2; the rest pass."""
    dims = rot["dims"]
    f, mult = rotary_frequencies(rot)
    out = x.clone()
    half = dims // 2
    for t in range(x.shape[0]):
        for i in range(half):
            a = float(pos[t]) * f[i]
            c, s = math.cos(a) * mult, math.sin(a) * mult
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------------------- mixers
def latent_attention(h, W, p, mx, eps, pos):
    """Queries through a normalised latent; keys and values rebuilt per head from one normalised latent per token plus one
    rotated key part shared by the heads; window of `mask.size` positions; a learned sink logit per head joins the
    softmax's denominator (no key, no value, not scaled)."""
    L = h.shape[0]
    H, d, r, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    cq = rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(L, H, d + r)
    z = h @ W[p + "dkv"].T
    c = rms(z[:, :R], eps) * W[p + "dkv.norm"]
    kr = rotate_half(z[:, None, R:], pos, mx["rot"])[:, 0]                        # [L, r]
    qr = rotate_half(q[:, :, d:], pos, mx["rot"])
    ku = (c @ W[p + "uk"].T).view(L, H, d)
    v = (c @ W[p + "uv"].T).view(L, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q[:, :, :d], ku) + torch.einsum("ihd,jd->hij", qr, kr)) * mx["scale"]
    dist = pos[:, None] - pos[None, :]
    ok = dist >= 0
    if mx.get("mask"):
        ok = ok & (dist < mx["mask"]["size"])
    s = s.masked_fill(~ok[None], float("-inf"))
    if p + "sink" in W:
        s = torch.cat([s, W[p + "sink"].view(H, 1, 1).expand(H, L, 1)], -1)
    pr = torch.softmax(s, -1)[..., :L]
    o = torch.einsum("hij,jhv->ihv", pr, v).reshape(L, H * dv)
    return o @ W[p + "o"].T


def biased_attention(h, W, p, mx, eps, pos):
    """Grouped-query softmax attention whose q and k pass a short causal convolution and then an RMS norm per head with a
    weight over the head's channels; the values are the convolved keys BEFORE their norm; the score loses
    slope_n (i - j) with slope_n = 2^(-8 (n + 1) / heads); causal, no positions otherwise."""
    L = h.shape[0]
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    q = short_conv(h @ W[p + "q"].T, W[p + "q.conv"]).view(L, H, d)
    k = short_conv(h @ W[p + "k"].T, W[p + "k.conv"]).view(L, G, d)
    v = k
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    rep = H // G
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, 1)) * mx["scale"]
    dist = (pos[:, None] - pos[None, :]).to(F64)
    slope = torch.tensor([2.0 ** (-8.0 * (n + 1) / H) for n in range(H)], dtype=F64)
    s = s - slope[:, None, None] * dist[None]
    s = s.masked_fill((dist < 0)[None], float("-inf"))
    pr = torch.softmax(s, -1)
    o = torch.einsum("hij,jhv->ihv", pr, v.repeat_interleave(rep, 1)).reshape(L, -1)
    return o @ W[p + "o"].T


def delta_rule(h, W, p, mx, eps):
    """Gated delta rule with one decay per head.  q, k, v pass a causal convolution and silu; q, k become unit vectors per
    head (x / sqrt(sum x^2 + 1e-6)), q times dim^-1/2.  Per token and head: S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  The read-out is divided by its RMS per head, weighted, gated by silu(W_g h) and projected."""
    L = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    rep = H // G
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(L, G, d)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(L, G, d)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(L, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                          # [L, H]
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(L, H, dv, dtype=F64)
    for t in range(L):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * W[p + "norm"]
    o = o.reshape(L, H * dv) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ----------------------------------------------------------------------------------------------- feed-forwards
def poly_norm_ff(h, W, p, eps):
    """W_down (a N(z) + b N(z^2) + c N(z^3) + e), z = W_up h, powers element by element, N = division of the token's vector
    by its root mean square."""
    z = h @ W[p + "up"].T
    a, b, c, e = [float(x) for x in W[p + "act"]]
    y = a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e
    return y @ W[p + "down"].T


def gated_expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def routed_ff(h, W, p, mlp):
    """Every token uses the `top` experts of largest router logit, weighted by the softmax over those logits alone; a
    shared expert runs for every token, times sigmoid(W_sg h)."""
    L = h.shape[0]
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ W[p + "router"].T
    val, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(val, -1)
    out = torch.zeros(L, W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(L):
        for j in range(top):
            out[t] += w[t, j] * gated_expert(h[t:t + 1], W, f"{p}e{int(idx[t, j])}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ W[p + "shared.sg"].T) * gated_expert(h, W, p + "shared.")
    return out


# ----------------------------------------------------------------------------------------------- the model
def mixer(cfg, W, i, x, pos):
    ly = cfg["layers"][i]
    p, mx, eps = f"l{i}.mix.", ly["mixer"], cfg["norm"]["eps"]
    if ly["type"] == "latent_attention":
        return latent_attention(x, W, p, mx, eps, pos)
    if ly["type"] == "attention":
        return biased_attention(x, W, p, mx, eps, pos)
    if ly["type"] == "delta":
        return delta_rule(x, W, p, mx, eps)
    raise ValueError(ly["type"])


def feed_forward(cfg, W, i, x):
    mlp = cfg["layers"][i]["mlp"]
    p = f"l{i}.mlp."
    if mlp["kind"] == "dense":
        return poly_norm_ff(x, W, p, cfg["norm"]["eps"])
    return routed_ff(x, W, p, mlp)


def forward(cfg, W, tokens, stream=None):
    """Logits [L, vocab] of one sequence; `stream` (a list) receives what every layer hands on."""
    eps, groups, m = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["residual_mult"]
    pos = torch.arange(len(tokens))
    x = W["embed"][torch.tensor(tokens)]
    hist = [x]
    for i, ly in enumerate(cfg["layers"]):
        x = x + m * group_rms(mixer(cfg, W, i, x, pos), groups, eps) * W[f"l{i}.norm1"]
        if ly.get("mlp") is not None:
            x = x + m * group_rms(feed_forward(cfg, W, i, x), groups, eps) * W[f"l{i}.norm2"]
        hist.append(x)
        a = W[f"l{i}.dwa"]
        x = sum(a[j] * hist[j] for j in range(i + 2))
        if stream is not None:
            stream.append(x.clone())
    return (group_rms(x, groups, eps) * W["final.norm"]) @ W["head"].T


# ----------------------------------------------------------------------------------------------- test models
def latent_layer(heads=4, dim=8, rot_dim=8, vdim=16, kv_rank=24, q_rank=16, window=20, base=10000.0, scale=0.2,
                 scaling=(4.0, 64, 8.0, 1.0), mlp="moe"):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
          "scale": scale, "rot": rot}
    if window:
        mx["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def attention_layer(heads=4, kv_heads=2, dim=16, conv=3, scale=0.25, mlp="dense"):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv,
                                           "scale": scale}, "mlp": mlp}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=8, conv=4, mlp="moe"):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp}


def make_config(layers, width=32, vocab=96, ff=48, experts=5, top=2, expert_ff=24, shared_ff=16, eps=1e-5, groups=4,
                residual_mult=0.5):
    out = []
    for ly in layers:
        ly = json.loads(json.dumps(ly))
        if ly["mlp"] == "dense":
            ly["mlp"] = {"kind": "dense", "ff": ff}
        elif ly["mlp"] == "moe":
            ly["mlp"] = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}}
            if shared_ff:
                ly["mlp"]["shared"] = {"ff": shared_ff}
        out.append(ly)
    return {"architecture": "Domorax", "vocab": vocab, "width": width, "layers": out,
            "norm": {"eps": eps, "groups": groups}, "residual_mult": residual_mult}


def random_weights(cfg, seed=0):
    """Tensors by checkpoint name, bf16-representable float32 (int tables none).  Norm weights around one, projections
    scaled so that activations stay of order one, decays spread between fast and slow, sinks of either sign."""
    g = torch.Generator().manual_seed(seed)
    Wd = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s / math.sqrt(i))).bfloat16().float()

    def vec(n, mean=0.0, std=1.0):
        return (mean + std * torch.randn(n, generator=g)).bfloat16().float()

    W = {"embed": vec(cfg["vocab"] * Wd).view(cfg["vocab"], Wd), "head": mat(cfg["vocab"], Wd), "final.norm": vec(Wd, 1.0, 0.2)}
    for i, ly in enumerate(cfg["layers"]):
        p, mx = f"l{i}.mix.", ly["mixer"]
        W[f"l{i}.norm1"] = vec(Wd, 1.0, 0.2)
        W[f"l{i}.dwa"] = (torch.cat([vec(i + 1, 0.0, 0.3), vec(1, 1.0, 0.1)]))
        if ly["type"] == "latent_attention":
            H, d, r, dv, R, Q = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            W[p + "dq"], W[p + "dq.norm"], W[p + "uq"] = mat(Q, Wd), vec(Q, 1.0, 0.2), mat(H * (d + r), Q, 2.0)
            W[p + "dkv"], W[p + "dkv.norm"] = mat(R + r, Wd, 2.0), vec(R, 1.0, 0.2)
            W[p + "uk"], W[p + "uv"] = mat(H * d, R, 2.0), mat(H * dv, R)
            W[p + "sink"] = vec(H, 0.0, 1.5)
            W[p + "o"] = mat(Wd, H * dv)
        elif ly["type"] == "attention":
            H, G, d, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["conv"]
            W[p + "q"], W[p + "k"] = mat(H * d, Wd), mat(G * d, Wd)
            W[p + "q.conv"], W[p + "k.conv"] = vec(H * d * taps, 0.3, 0.5).view(H * d, taps), vec(G * d * taps, 0.3, 0.5).view(G * d, taps)
            W[p + "q.norm"], W[p + "k.norm"] = vec(d, 1.0, 0.3), vec(d, 1.0, 0.3)
            W[p + "o"] = mat(Wd, H * d)
        else:
            H, G, d, dv, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
            for n, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                W[p + n] = mat(rows, Wd)
                W[p + n + ".conv"] = vec(rows * taps, 0.3, 0.5).view(rows, taps)
            W[p + "b"], W[p + "a"], W[p + "g"] = mat(H, Wd), mat(H, Wd), mat(H * dv, Wd)
            W[p + "A_log"], W[p + "dt_bias"] = vec(H, -1.0, 1.0), vec(H, 0.0, 1.0)
            W[p + "norm"] = vec(dv, 1.0, 0.2)
            W[p + "o"] = mat(Wd, H * dv)
        mlp = ly.get("mlp")
        if mlp is None:
            continue
        q = f"l{i}.mlp."
        W[f"l{i}.norm2"] = vec(Wd, 1.0, 0.2)
        if mlp["kind"] == "dense":
            W[q + "up"], W[q + "down"], W[q + "act"] = mat(mlp["ff"], Wd), mat(Wd, mlp["ff"]), vec(4, 0.3, 0.6)
        else:
            f = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                W[f"{q}e{e}.gate"], W[f"{q}e{e}.up"], W[f"{q}e{e}.down"] = mat(f, Wd), mat(f, Wd), mat(Wd, f)
            W[q + "router"] = mat(mlp["router"]["experts"], Wd, 2.0)
            if mlp.get("shared"):
                f = mlp["shared"]["ff"]
                W[q + "shared.gate"], W[q + "shared.up"], W[q + "shared.down"] = mat(f, Wd), mat(f, Wd), mat(Wd, f)
                W[q + "shared.sg"] = mat(1, Wd)
    return W


def to64(W):
    return {k: v.to(F64) for k, v in W.items()}


def write_checkpoint(folder, cfg, W):
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in W.items()}, os.path.join(folder, "model.safetensors"))
    return str(folder)
