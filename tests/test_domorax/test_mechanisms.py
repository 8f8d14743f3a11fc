"""Every mechanism of the Domorax family alone: the framework's module on the framework's step runtime (sm_100a kernels on
the `gpu` tier, their PyTorch paths on the plumbing tier) against the float64 oracle's function of the same mechanism.
Inputs and weights are made so that a fault shows: a key that one query singles out among hundreds, keys just inside and
just outside the window and on a page's border, sink scores that outweigh the keys, decays of almost one and almost zero,
portions shorter than the convolution, widths that take the scalar paths."""
import pytest
import torch

from colossalai_b200.inference.modeling.kv_runtime import PagedKVRuntime
from colossalai_b200.models.domorax import DomoraxForCausalLM, convert_domorax_state_dict, domorax_config
from colossalai_b200.ops import mixers as M
from colossalai_b200.ops import moe as MO

from . import oracle as O

TIERS = ["plumbing", pytest.param("gpu", marks=pytest.mark.gpu)]
F64 = torch.float64
BS = 8           # page size of the scratch runtime
WIDTH = 40


def _dev(tier):
    if tier == "gpu" and not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return "cuda" if tier == "gpu" else "cpu"


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def _close(got, want, tol):
    err = (got.double().cpu() - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err < tol, f"relative error {err:.3e}"


def _layer(layer, dev, width=WIDTH, seed=0, edit=None, dtype=torch.float32, **kw):
    """One-layer model of `layer`: (framework layer module, its config, oracle weights, hf config)."""
    hf = O.make_config([layer], width=width, **kw)
    W = O.random_weights(hf, seed=seed)
    if edit:
        edit(W)
        W = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    cfg = domorax_config(hf, {k: tuple(v.shape) for k, v in W.items()})
    model = DomoraxForCausalLM(cfg)
    missing, unexpected = model.load_state_dict(convert_domorax_state_dict(W, cfg), strict=False)
    assert not missing and not unexpected
    return model.to(dtype).to(dev).eval().model.layers[0], cfg, O.to64(W), hf


def _steps(mixer, cfg, h, cuts, dev, dtype=torch.float32, batch_with=None):
    """Run h [L, width] through the mixer in portions of the given sizes on a scratch runtime (pages of BS tokens, two
    slots; the sequence under test sits in slot 1 and its pages are handed out back to front).  `batch_with`: another
    sequence's input that shares every step (a fresh one-step prompt each time)."""
    L = h.shape[0]
    rt = PagedKVRuntime.scratch(cfg, 2, L + 64, dev, dtype, block_size=BS)
    for st in rt.states:                                   # recycled slots are never cleared: leave rubbish in them
        for t in (st or {}).values():
            t.fill_(3.0)
    per = (L + 64 + BS - 1) // BS
    tables = torch.stack([torch.arange(per, dtype=torch.int32), torch.arange(2 * per - 1, per - 1, -1, dtype=torch.int32)])
    out, at = [], 0
    with torch.inference_mode():
        for n in cuts:
            if batch_with is not None:
                rt.set_ragged_step(tables, [batch_with.shape[0], n], [0, at], [0, 1], dev)
                x = torch.cat([batch_with, h[at:at + n]]).to(dev).to(dtype)
                out.append(mixer(x, None, None, rt)[batch_with.shape[0]:])
            else:
                rt.set_ragged_step(tables[1:], [n], [at], [1], dev)
                out.append(mixer(h[at:at + n].to(dev).to(dtype), None, None, rt))
            at += n
    assert at == L
    return torch.cat(out)


def _cuts(L, sizes):
    out, at = [], 0
    for n in sizes:
        n = min(n, L - at)
        if n > 0:
            out.append(n)
            at += n
    return out + [1] * (L - at)


CUTS = lambda L: ([L], [1] * L, _cuts(L, [2, 3, 2, 9, 1, 1, 17, 2, 40]), _cuts(L, [L - 3]))


# ------------------------------------------------------------------------------------------------ latent attention
def _latent_probe(W):
    """The query's latent equals the key's latent and the unrotated query rows equal the unrotated key rows, the rotated
    query rows are zero: a query scores the key made from the same input with |k|^2 > 0, all others at random."""
    p = "l0.mix."
    R = W[p + "dkv.norm"].numel()
    H = W[p + "sink"].numel()
    d = W[p + "uk"].shape[0] // H
    W[p + "dq"] = W[p + "dkv"][:R].clone()
    W[p + "dq.norm"] = W[p + "dkv.norm"].clone()
    uq = W[p + "uq"].view(H, -1, R)
    uq[:, :d] = W[p + "uk"].view(H, d, R)
    uq[:, d:] = 0.0


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("window,probe", [(20, 41), (20, 40), (BS + 1, 52), (BS, 52), (0, 2), (1, 60), (100, 0)])
def test_latent_attention_at_the_window_edges(tier, window, probe):
    """The last query (position 60) repeats the input of position `probe`: that key outscores all others IF the window
    lets the query see it.  Probes sit on the first position inside the window, one before it, on a page border, far back
    without a window, on the query itself - in whole prompts, in portions, decoded token by token, beside another request.
    Sink scores of both signs, one of them above every key's score of its head."""
    dev = _dev(tier)
    L = 61
    layer = O.latent_layer(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=16, q_rank=16, window=window, scale=0.6)

    def edit(W):
        _latent_probe(W)
        W["l0.mix.sink"] = torch.tensor([-2.0, 0.5, 9.0])
    mod, cfg, W, hf = _layer(layer, dev, seed=1, edit=edit)
    h = _rand(L, WIDTH, seed=2)
    h[L - 1] = h[probe]
    want = O.latent_attention(h.to(F64), W, "l0.mix.", hf["layers"][0]["mixer"], 1e-5, torch.arange(L))
    for cuts in CUTS(L):
        _close(_steps(mod.self_attn, cfg, h, cuts, dev), want, 3e-5)
    _close(_steps(mod.self_attn, cfg, h, _cuts(L, [5, 30]), dev, batch_with=_rand(19, WIDTH, seed=3)), want, 3e-5)
    # the probe decides the last row: without it the row differs
    other = O.latent_attention(torch.cat([h[:-1], h[5:6]]).to(F64), W, "l0.mix.", hf["layers"][0]["mixer"], 1e-5,
                               torch.arange(L))
    seen = window == 0 or L - 1 - probe < window
    assert ((other[-1] - want[-1]).abs().max() > 1e-3) or not seen


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("scaling", [(4.0, 64, 8.0, 1.0), None, (1.5, 16, 4.0, 2.0)])
def test_latent_attention_far_key_with_rotated_parts(tier, scaling):
    """350 positions without a window; the rotated query and key parts are in play (random weights), with frequencies
    stretched for long contexts or plain."""
    dev = _dev(tier)
    L = 350
    layer = O.latent_layer(heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=24, q_rank=8, window=0, scale=0.3, base=200.0,
                           scaling=scaling)
    mod, cfg, W, hf = _layer(layer, dev, seed=4)
    h = _rand(L, WIDTH, seed=5)
    h[L - 1] = h[3]
    want = O.latent_attention(h.to(F64), W, "l0.mix.", hf["layers"][0]["mixer"], 1e-5, torch.arange(L))
    for cuts in ([L], _cuts(L, [L - 30]), _cuts(L, [2, 130, 2, 180, 7])):
        _close(_steps(mod.self_attn, cfg, h, cuts, dev), want, 3e-5)


@pytest.mark.parametrize("tier", TIERS)
def test_rotary_table_with_stretched_frequencies(tier):
    dev = _dev(tier)
    for dims, base, sc in [(16, 1e4, (4.0, 64, 8.0, 1.0)), (32, 5e4, (2.0, 512, 32.0, 1.0)), (8, 100.0, None),
                           (4, 1e3, (8.0, 32, 1.0, 1.0))]:
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        x = _rand(6, 2, dims + 3, seed=dims).to(F64)
        pos = torch.tensor([0, 1, 2, 300, 1023, 4000])
        want = O.rotate_half(x, pos, rot)
        table = M.rotary_table(4001, dims, base, dev, sc)
        src = x.float().reshape(6, -1).to(dev)
        dst = torch.zeros_like(src)
        M.rotary_half(src, dst, 2, dims + 3, 0, dims + 3, 0, dims + 3, dims, table, pos.to(torch.int32).to(dev))
        _close(dst.view(6, 2, dims + 3), want, 2e-5)


# ------------------------------------------------------------------------------------------------ convolved attention
def _tie_q_to_k(W):
    p = "l0.mix."
    rep = W[p + "q"].shape[0] // W[p + "k"].shape[0]
    G = W[p + "k"].shape[0] // W[p + "k.norm"].numel()
    d = W[p + "k.norm"].numel()
    W[p + "q"] = W[p + "k"].view(G, 1, d, -1).expand(G, rep, d, -1).reshape(G * rep * d, -1).clone()
    W[p + "q.conv"] = W[p + "k.conv"].view(G, 1, d, -1).expand(G, rep, d, -1).reshape(G * rep * d, -1).clone()
    W[p + "q.norm"] = W[p + "k.norm"].clone()


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("heads,kv,dim,conv,probe", [(4, 2, 16, 3, 5), (3, 3, 8, 4, 290), (2, 1, 24, 2, 3 * BS), (1, 1, 40, 1, 7)])
def test_convolved_attention_finds_a_far_key(tier, heads, kv, dim, conv, probe):
    """300 positions; the inputs in front of the last query repeat those in front of position `probe`, so that the
    convolved query equals that position's convolved key (tied weights).  The last head's slope is small enough for a far
    key to win; the first head's slope buries it - both show in the output."""
    dev = _dev(tier)
    L = 300
    layer = O.attention_layer(heads=heads, kv_heads=kv, dim=dim, conv=conv, scale=2.0)
    mod, cfg, W, hf = _layer(layer, dev, seed=6, edit=_tie_q_to_k)
    h = _rand(L, WIDTH, seed=7)
    for j in range(conv):
        h[L - 1 - j] = h[probe - j]
    want = O.biased_attention(h.to(F64), W, "l0.mix.", hf["layers"][0]["mixer"], 1e-5, torch.arange(L))
    for cuts in ([L], _cuts(L, [L - 20]), _cuts(L, [2, 1, 130, 2, 140, 7])):
        _close(_steps(mod.self_attn, cfg, h, cuts, dev), want, 3e-5)
    _close(_steps(mod.self_attn, cfg, h, _cuts(L, [1, 2, 250]), dev, batch_with=_rand(9, WIDTH, seed=3)), want, 3e-5)


@pytest.mark.parametrize("tier", TIERS)
def test_convolved_attention_first_tokens_and_short_portions(tier):
    dev = _dev(tier)
    L = 37
    layer = O.attention_layer(heads=4, kv_heads=2, dim=8, conv=4, scale=0.7)
    mod, cfg, W, hf = _layer(layer, dev, seed=8)
    h = _rand(L, WIDTH, seed=9)
    want = O.biased_attention(h.to(F64), W, "l0.mix.", hf["layers"][0]["mixer"], 1e-5, torch.arange(L))
    for cuts in CUTS(L):
        got = _steps(mod.self_attn, cfg, h, cuts, dev)
        _close(got[:5], want[:5], 3e-5)
        _close(got, want, 3e-5)


@pytest.mark.parametrize("tier", TIERS)
def test_head_norm_op(tier):
    dev = _dev(tier)
    T, Ha, Hb, d = 7, 3, 2, 12
    x = _rand(T, (Ha + Hb) * d + 5, seed=1, scale=3.0)
    wa, wb = _rand(d, seed=2) + 1.0, _rand(d, seed=3) + 1.0
    got = M.head_rms_norm(x.to(dev), Ha, Hb, d, wa.to(dev), wb.to(dev), 1e-5)
    y = O.rms(x[:, : (Ha + Hb) * d].to(F64).view(T, Ha + Hb, d), 1e-5)
    want = torch.cat([y[:, :Ha] * wa.to(F64), y[:, Ha:] * wb.to(F64)], 1).reshape(T, -1)
    _close(got, want, 3e-6)


# ------------------------------------------------------------------------------------------------ delta rule
@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("heads,kv,dim,vdim,conv", [(4, 2, 16, 8, 4), (1, 1, 40, 24, 2), (3, 3, 8, 40, 3), (2, 1, 72, 16, 1)])
def test_delta_rule_with_slow_and_fast_heads(tier, heads, kv, dim, vdim, conv):
    """A_log from -5 (decay of almost one: the state remembers the whole sequence) to +2 (almost zero), write strengths
    pushed towards both ends."""
    dev = _dev(tier)
    L = 80

    def edit(W):
        W["l0.mix.A_log"] = torch.linspace(-5, 2, heads)
        W["l0.mix.dt_bias"] = torch.linspace(-2, 2, heads)
        W["l0.mix.b"] *= 4.0
    layer = O.delta_layer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv)
    mod, cfg, W, hf = _layer(layer, dev, seed=10, edit=edit)
    h = _rand(L, WIDTH, seed=11)
    want = O.delta_rule(h.to(F64), W, "l0.mix.", hf["layers"][0]["mixer"], 1e-5)
    for cuts in CUTS(L):
        _close(_steps(mod.self_attn, cfg, h, cuts, dev), want, 5e-5)
    _close(_steps(mod.self_attn, cfg, h, _cuts(L, [1, 1, 2, 30]), dev, batch_with=_rand(3, WIDTH, seed=3)), want, 5e-5)


# ------------------------------------------------------------------------------------------------ feed-forwards, norms, history
@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("ff", [48, 50, 7])
def test_normalised_power_feed_forward(tier, ff):
    dev = _dev(tier)
    mod, cfg, W, hf = _layer(O.delta_layer(mlp="dense"), dev, seed=12, ff=ff,
                             edit=lambda W: W.__setitem__("l0.mlp.act", torch.tensor([0.75, -0.5, 0.25, 0.125])))
    h = _rand(21, WIDTH, seed=13, scale=2.0)
    with torch.inference_mode():
        got = mod.mlp(h.to(dev))
    _close(got, O.poly_norm_ff(h.to(F64), W, "l0.mlp.", 1e-5), 2e-5)
    z = _rand(5, ff + 3, seed=14, scale=3.0)[:, 3:]
    coef = torch.tensor([0.3, 1.5, -0.7, 0.2])
    zz = z.to(F64)
    want = 0.3 * O.rms(zz, 1e-6) + 1.5 * O.rms(zz ** 2, 1e-6) - 0.7 * O.rms(zz ** 3, 1e-6) + 0.2
    _close(M.poly_norm(z.to(dev), coef.to(dev), 1e-6), want, 3e-6)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("experts,top,shared", [(5, 2, 16), (1, 1, 8), (6, 6, 0), (4, 1, 24), (7, 3, 16)])
def test_routed_feed_forward(tier, experts, top, shared):
    """Random inputs keep the router's choices apart (no test rests on a close call): the weights are the softmax over the
    chosen logits, the shared expert sits behind its sigmoid gate or is absent."""
    dev = _dev(tier)
    mod, cfg, W, hf = _layer(O.delta_layer(mlp="moe"), dev, seed=15, experts=experts, top=top, shared_ff=shared,
                             edit=lambda W: W.__setitem__("l0.mlp.router", W["l0.mlp.router"] * 3.0))
    h = _rand(23, WIDTH, seed=16, scale=1.5)
    with torch.inference_mode():
        got = mod.mlp(h.to(dev))
    if isinstance(got, tuple):
        assert got[1] is None
        got = got[0]
    assert got.dtype == torch.float32
    _close(got, O.routed_ff(h.to(F64), W, "l0.mlp.", hf["layers"][0]["mlp"]), 2e-5)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("W,groups", [(48, 4), (50, 5), (1024, 2), (36, 1), (33, 3)])
def test_grouped_norm_into_the_stream(tier, W, groups):
    dev = _dev(tier)
    T = 5
    x, y, w = _rand(T, W, seed=1), _rand(T, W + 8, seed=2, scale=5.0)[:, 8:], _rand(W, seed=3) + 1.0
    y = y * torch.linspace(0.01, 3.0, W)                    # groups of very unequal size
    want = x.to(F64) + 0.5 * O.group_rms(y.to(F64), groups, 1e-5) * w.to(F64)
    xs = x.clone().to(dev)
    h = M.rms_norm_residual(xs, y.to(dev), w.to(dev), 1e-5, mult=0.5, groups=groups)
    _close(xs, want, 3e-6)
    _close(h, want, 3e-6)
    _close(M.rms_norm_f32in(y.to(dev), w.to(dev), 1e-5, groups=groups), O.group_rms(y.to(F64), groups, 1e-5) * w.to(F64), 3e-6)


@pytest.mark.parametrize("tier", TIERS)
def test_weighted_sum_over_the_stream_history(tier):
    dev = _dev(tier)
    for T, W, n in [(5, 48, 3), (3, 33, 1), (2, 1024, 6)]:
        hist = _rand(8, T, W, seed=T).to(dev)
        coef = _rand(8, seed=W)
        want = sum(coef[j].to(F64) * hist[j].double().cpu() for j in range(n))
        h = M.depth_mix(hist, n, coef.to(dev), hist[n], cast_dtype=torch.bfloat16)
        _close(hist[n], want, 3e-6)
        _close(h, want, 1e-2)
        assert h.dtype == torch.bfloat16


@pytest.mark.parametrize("tier", TIERS)
def test_combine_with_a_gated_shared_row(tier):
    dev = _dev(tier)
    T, k, H = 6, 2, 24
    rows, extra = _rand(T * k, H, seed=1), _rand(T, H, seed=2)
    row_of = torch.randperm(T * k, generator=torch.Generator().manual_seed(3)).view(T, k)
    w, g = _rand(T, k, seed=4).abs(), _rand(T, 3, seed=5)[:, 1]
    want = sum(w[:, j:j + 1].to(F64) * rows[row_of[:, j]].to(F64) for j in range(k)) + \
        torch.sigmoid(g.to(F64))[:, None] * extra.to(F64)
    got = MO.gather_combine(rows.to(dev), row_of.to(dev), w.to(dev), extra=extra.to(dev), extra_gate=g.to(dev))
    _close(got, want, 3e-6)


# ------------------------------------------------------------------------------------------------ the kernels against each other
@pytest.mark.gpu
@pytest.mark.parametrize("window,L,dim,vdim,same", [(0, 300, 32, 32, False), (24, 300, 64, 64, False), (200, 460, 40, 24, True),
                                                    (130, 700, 160, 128, True), (72, 900, 64, 64, False)])
def test_tensor_core_attention_against_the_exact_kernel(window, L, dim, vdim, same):
    """16-bit pages through the tensor-core kernel - windows, learned sinks, distance slopes, values inside the key rows,
    long portions whose few row tiles split their keys over CTAs, decoded tokens whose window starts inside a key chunk -
    row by row against the exact kernel on the same pages."""
    dev = _dev("gpu")
    H, G, bs = 4, 1 if same else 2, 16
    nb = L // bs + 1
    kc = _rand(nb, bs, G, dim, seed=1).to(dev).to(torch.bfloat16)
    vc = kc if same else _rand(nb, bs, G, vdim, seed=2).to(dev).to(torch.bfloat16)
    tables = torch.arange(nb, dtype=torch.int32, device=dev).view(1, -1)
    sinks = torch.tensor([-1.0, 0.0, 2.0, 6.0], device=dev)
    slopes = None if same else M.distance_slopes(H).to(dev)
    for q_len in (L, 1, 5, 130):
        meta = M.RaggedMeta.build([q_len], [L - q_len], [0], dev)
        q = _rand(q_len, H * dim, seed=3, scale=1.0).to(dev).to(torch.bfloat16)
        kw = dict(sink=True, sink_values=sinks, slopes=slopes, window=window, vdim=vdim if same else None)
        exact = M.paged_bias_attention(q, kc, vc, tables, meta, 0.2, tensor_cores=False, **kw).float()
        got = M.paged_bias_attention(q, kc, vc, tables, meta, 0.2, tensor_cores=True, wide_weights=True, **kw).float()
        rows = (got - exact).norm(dim=-1) / exact.norm(dim=-1).clamp_min(1e-3)
        assert rows.max() < 2e-2, f"q_len {q_len}, row {int(rows.argmax())}: relative error {float(rows.max()):.3e}"
