"""Every mechanism of the Pogorax family alone: the framework's mixer module on the framework's step runtime (sm_100a
kernels on the `gpu` tier, their PyTorch paths on the plumbing tier) against the float64 oracle's function of the same
mechanism.  Inputs and weights are made so that a fault shows: a key that one query singles out among hundreds, keys on
both sides of a mask block's and a page's border, gates that jump the running maximum, decays of almost one and almost
zero, portions shorter than the convolution, widths that take the scalar paths."""
import math

import pytest
import torch

from colossalai_b200.inference.modeling.kv_runtime import PagedKVRuntime
from colossalai_b200.models.pogorax import PogoraxForCausalLM, convert_pogorax_state_dict, pogorax_config
from colossalai_b200.ops import mixers as M

from . import oracle as O

TIERS = ["plumbing", pytest.param("gpu", marks=pytest.mark.gpu)]
F64 = torch.float64
BS = 8           # page size of the scratch runtime


def _dev(tier):
    if tier == "gpu" and not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return "cuda" if tier == "gpu" else "cpu"


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def _close(got, want, tol):
    err = (got.double().cpu() - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err < tol, f"relative error {err:.3e}"


def _layer(layer, dev, width=48, seed=0, edit=None, dtype=torch.float32):
    """One-layer model of `layer`: (framework mixer module, its config, oracle weights, hf config)."""
    hf = O.make_config([layer], width=width)
    W = O.random_weights(hf, seed=seed)
    if edit:
        edit(W)
        W = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    shapes = {k: tuple(v.shape) for k, v in W.items()}
    cfg = pogorax_config(hf, shapes)
    model = PogoraxForCausalLM(cfg)
    missing, unexpected = model.load_state_dict(convert_pogorax_state_dict(W, cfg), strict=False)
    assert not missing and not unexpected
    return model.to(dtype).to(dev).eval().model.layers[0].self_attn, cfg, O.to64(W), hf


def _steps(mixer, cfg, h, cuts, dev, dtype=torch.float32, batch_with=None):
    """Run h [L, width] through the mixer in portions of the given sizes on a scratch runtime (pages of BS tokens, two
    slots; the sequence under test sits in slot 1 and its pages are handed out back to front).  `batch_with`: another
    sequence's input that shares every step (a fresh one-step prompt each time)."""
    L = h.shape[0]
    rt = PagedKVRuntime.scratch(cfg, 2, L + 64, dev, dtype, block_size=BS)
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


# ------------------------------------------------------------------------------------------------ attention
def _tie_queries_to_keys(p, heads):
    """q weights = k weights for every head: a query and a key from the same input score |W_k h|^2 > 0."""
    def edit(W):
        W[p + "q"] = W[p + "k"].repeat(heads, 1)
    return edit


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("mask,probe", [(12, 36), (12, 35), (BS, 16), (20, 59), (0, 3)])
def test_block_masked_gated_attention_at_the_edges(tier, mask, probe):
    """The last query repeats the input of position `probe`, strongly: with tied q / k weights that key outscores all
    others IF the mask lets the query see it.  Probes sit on the first position of the query's block, one before it, on a
    page border, far back without a mask - in whole prompts, in portions and decoded token by token."""
    dev = _dev(tier)
    L = 61                                                 # the last query sits at position 60
    layer = O.gated_pair_layer(heads=3, kv_heads=1, dim=16, vdim=24, scale=0.5, mask=mask)
    mixer, cfg, W, hf = _layer(layer, dev, seed=1, edit=_tie_queries_to_keys("l0.mix.left.", 3))
    h = _rand(L, 48, seed=2)
    h[probe] *= 3.0
    h[L - 1] = h[probe]
    att = mixer.parts[0]
    want = O.softmax_attention(h.to(F64), W, "l0.mix.left.", hf["layers"][0]["mixer"]["left"], 1e-5, list(range(L)),
                               unit_norm=False, gated=True)
    for cuts in CUTS(L):
        _close(_steps(att, cfg, h, cuts, dev), want, 2e-5)
    _close(_steps(att, cfg, h, _cuts(L, [5, 30]), dev, batch_with=_rand(19, 48, seed=3)), want, 2e-5)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("rot_dims,kv", [(8, 1), (16, 2), (0, 4)])
def test_rotary_unit_norm_attention_finds_a_far_key(tier, rot_dims, kv):
    """Causal attention over 400 positions: the last query repeats position 3's input.  Unit-RMS heads bound the scores, so
    the scale is large enough for one key to stand out."""
    dev = _dev(tier)
    L = 400
    layer = O.rotary_pair_layer(heads=4, kv_heads=kv, dim=16, vdim=8, scale=1.5, rot_dims=rot_dims, base=300.0)
    mixer, cfg, W, hf = _layer(layer, dev, seed=4)
    h = _rand(L, 48, seed=5)
    h[L - 1] = h[3]
    att = mixer.parts[0]
    want = O.softmax_attention(h.to(F64), W, "l0.mix.left.", hf["layers"][0]["mixer"]["left"], 1e-5, list(range(L)),
                               unit_norm=True, gated=False)
    for cuts in ([L], _cuts(L, [L - 40]), _cuts(L, [2, 130, 2, 200, 7])):
        _close(_steps(att, cfg, h, cuts, dev), want, 3e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("mask,L", [(0, 300), (24, 300), (200, 460), (130, 700)])
def test_tensor_core_attention_row_by_row(mask, L):
    """16-bit serving through the tensor-core kernel, every output row against the oracle: causal and block-masked, long
    portions whose few row tiles split their keys over CTAs (key chunks that a mask block's start cuts), decoded tokens."""
    dev = _dev("gpu")
    layer = O.gated_pair_layer(heads=4, kv_heads=2, dim=32, vdim=64, scale=0.4, mask=mask)
    mixer, cfg, W, hf = _layer(layer, dev, seed=6, dtype=torch.bfloat16)
    h = _rand(L, 48, seed=7).to(torch.bfloat16).float()
    want = O.softmax_attention(h.to(F64), W, "l0.mix.left.", hf["layers"][0]["mixer"]["left"], 1e-5, list(range(L)),
                               unit_norm=False, gated=True)
    for cuts in ([L], _cuts(L, [L - 20]), _cuts(L, [100, 3, 150])):
        got = _steps(mixer.parts[0], cfg, h, cuts, dev, dtype=torch.bfloat16).double().cpu()
        rows = (got - want).norm(dim=-1) / want.norm(dim=-1)
        assert rows.max() < 4e-2, f"row {int(rows.argmax())}: relative error {float(rows.max()):.3e}"


@pytest.mark.gpu
def test_two_term_weights_tighten_the_weighted_sum():
    """The same pages through the tensor-core kernel with one-term and two-term softmax weights, against the exact
    kernel: the second term brings the weighted sum several times closer."""
    dev = _dev("gpu")
    H, G, d, bs, L = 4, 1, 64, 16, 520
    meta = M.RaggedMeta.build([L], [0], [0], dev)
    kc = _rand(L // bs + 1, bs, G, d, seed=1).to(dev).to(torch.bfloat16)
    vc = _rand(L // bs + 1, bs, G, d, seed=2).to(dev).to(torch.bfloat16)
    tables = torch.arange(L // bs + 1, dtype=torch.int32, device=dev).view(1, -1)
    q = _rand(L, H * d, seed=3, scale=2.0).to(dev).to(torch.bfloat16)
    exact = M.paged_bias_attention(q, kc, vc, tables, meta, 0.125, tensor_cores=False).float()
    err = {}
    for wide in (False, True):
        got = M.paged_bias_attention(q, kc, vc, tables, meta, 0.125, wide_weights=wide).float()
        err[wide] = float(((got - exact).norm(dim=-1) / exact.norm(dim=-1)).mean())
    assert err[True] < 0.5 * err[False], err


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("dims,width,interleaved", [(8, 8, True), (4, 12, True), (0, 6, True), (32, 40, False),
                                                    (6, 7, True)])
def test_rotary_pairs_and_unit_norm_op(tier, dims, width, interleaved):
    dev = _dev(tier)
    T, H = 9, 3
    x = _rand(T, H * width + 5, seed=1)
    pos = torch.tensor([0, 1, 2, 700, 701, 5, 31, 32, 4095], dtype=torch.int32)
    table = M.rotary_table(5000, dims, 1e4, dev) if dims else None
    y = x.clone().to(dev)
    M.rotary_unit_norm(y, H, width, dims, interleaved, table, pos.to(dev), 1e-5)
    heads = x[:, : H * width].view(T, H, width).to(F64)
    if interleaved:
        want = O.rotate_pairs(heads, pos.tolist(), dims, 1e4)
    else:                                                  # pairs (i, i + dims / 2): the same turn on regrouped channels
        order = [c for i in range(dims // 2) for c in (i, i + dims // 2)] + list(range(dims, width))
        want = torch.empty_like(heads)
        want[..., order] = O.rotate_pairs(heads[..., order], pos.tolist(), dims, 1e4)
    want = O.rms(want, 1e-5)
    _close(y[:, : H * width].view(T, H, width), want, 3e-6)
    assert torch.equal(y[:, H * width:].cpu(), x[:, H * width:])      # columns behind the heads are left alone


# ------------------------------------------------------------------------------------------------ recurrences
@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("heads,dim,vdim,cap", [(3, 8, 16, 6.0), (1, 40, 8, 2.0), (2, 16, 40, 15.0), (2, 72, 24, 4.0)])
def test_matrix_memory_with_gates_that_jump(tier, heads, dim, vdim, cap):
    """Input-gate biases from -8 to +8 and forget-gate biases down to -6: the running maximum is taken over by single
    tokens and decays back; the denominator's floor exp(-m) is active for the first tokens."""
    dev = _dev(tier)
    L = 70

    def edit(W):
        W["l0.mix.right.i.b"] = torch.linspace(-8, 8, heads)
        W["l0.mix.right.f.b"] = torch.linspace(-6, 4, heads)
        W["l0.mix.right.i"] *= 4.0
    layer = O.gated_pair_layer(m_heads=heads, m_dim=dim, m_vdim=vdim, cap=cap)
    mixer, cfg, W, hf = _layer(layer, dev, seed=8, edit=edit)
    h = _rand(L, 48, seed=9)
    want = O.matrix_memory(h.to(F64), W, "l0.mix.right.", hf["layers"][0]["mixer"]["right"], 1e-5)
    for cuts in CUTS(L):
        _close(_steps(mixer.parts[1], cfg, h, cuts, dev), want, 5e-5)
    _close(_steps(mixer.parts[1], cfg, h, _cuts(L, [5, 30]), dev, batch_with=_rand(11, 48, seed=3)), want, 5e-5)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("width,blocks,conv", [(32, 2, 4), (40, 1, 2), (24, 3, 3), (33, 1, 4)])
def test_linear_recurrent_unit_with_slow_and_fast_channels(tier, width, blocks, conv):
    """lam from -9 (decay of almost one: the state remembers the whole sequence) to +4 (almost zero)."""
    dev = _dev(tier)
    L = 90

    def edit(W):
        W["l0.mix.right.lam"] = torch.linspace(-9, 4, width)
    layer = O.rotary_pair_layer(width=width, blocks=blocks, conv=conv)
    mixer, cfg, W, hf = _layer(layer, dev, seed=10, edit=edit)
    h = _rand(L, 48, seed=11)
    want = O.linear_recurrent_unit(h.to(F64), W, "l0.mix.right.", hf["layers"][0]["mixer"]["right"])
    for cuts in CUTS(L):
        _close(_steps(mixer.parts[1], cfg, h, cuts, dev), want, 5e-5)
    _close(_steps(mixer.parts[1], cfg, h, _cuts(L, [1, 2, 40]), dev, batch_with=_rand(7, 48, seed=3)), want, 5e-5)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("heads,vdim,state,groups,parts,conv", [(4, 8, 16, 2, 2, 4), (1, 40, 24, 1, 1, 2),
                                                                (6, 8, 8, 6, 3, 3), (2, 24, 72, 1, 4, 4)])
def test_state_space_with_portions_shorter_than_the_convolution(tier, heads, vdim, state, groups, parts, conv):
    dev = _dev(tier)
    L = 64

    def edit(W):
        W["l0.mix.A_log"] = torch.linspace(-4, 1.5, heads)          # from almost no decay to a fast one
        W["l0.mix.dt_bias"] = torch.linspace(-3, 3, heads)
    layer = O.state_space_layer(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=parts, conv=conv)
    mixer, cfg, W, hf = _layer(layer, dev, seed=12, edit=edit)
    h = _rand(L, 48, seed=13)
    want = O.state_space(h.to(F64), W, "l0.mix.", hf["layers"][0]["mixer"], 1e-5)
    for cuts in CUTS(L):
        _close(_steps(mixer, cfg, h, cuts, dev), want, 5e-5)
    _close(_steps(mixer, cfg, h, _cuts(L, [1, 1, 2, 30]), dev, batch_with=_rand(3, 48, seed=3)), want, 5e-5)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("C,taps,act", [(24, 4, True), (7, 2, False), (40, 3, False), (16, 1, True)])
def test_convolution_with_bias_carries_its_window(tier, C, taps, act):
    dev = _dev(tier)
    L = 23
    x, w, b = _rand(L, C + 3, seed=1), _rand(C, taps, seed=2), _rand(C, seed=3)
    want = O.short_conv(x[:, 3:].to(F64), w.to(F64), b.to(F64))
    want = O.silu(want) if act else want
    for cuts in ([L], [1] * L, _cuts(L, [2, 1, 5, 1, 1, 9])):
        state = torch.full((3, max(taps - 1, 0), C), 7.0, device=dev)         # a recycled slot: never cleared
        got, at = [], 0
        for n in cuts:
            meta = M.RaggedMeta.build([n], [at], [2], dev)
            got.append(M.short_conv_silu(x.to(dev)[at:at + n, 3:], w.to(dev), state, meta, activation=act, bias=b.to(dev)))
            at += n
        _close(torch.cat(got), want, 3e-6)


# ------------------------------------------------------------------------------------------------ pair, norms, feed-forward
@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("kind", ["gated", "rotary"])
def test_pair_averages_the_normed_outputs(tier, kind):
    dev = _dev(tier)
    L = 33
    layer = O.gated_pair_layer(mask=10) if kind == "gated" else O.rotary_pair_layer()
    mixer, cfg, W, hf = _layer(layer, dev, seed=14)
    h = _rand(L, 48, seed=15)
    want = O.pair(h.to(F64), W, "l0.mix.", hf["layers"][0], 1e-5, list(range(L)))
    for cuts in ([L], _cuts(L, [2, 11, 1, 1, 7])):
        got = _steps(mixer, cfg, h, cuts, dev)
        assert got.dtype == torch.float32
        _close(got, want, 5e-5)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("W", [48, 50, 1024])
def test_mean_of_normed_tensors_and_gate_ops(tier, W):
    dev = _dev(tier)
    T = 5
    a, b = _rand(T, W, seed=1, scale=3.0), _rand(T, W + 8, seed=2, scale=0.01)[:, 8:]      # very unequal sizes
    wa, wb = _rand(W, seed=3) + 1.0, _rand(W, seed=4) + 1.0
    want = 0.5 * (O.rms(a.to(F64), 1e-6) * wa.to(F64) + O.rms(b.to(F64), 1e-6) * wb.to(F64))
    _close(M.norm_mean([a.to(dev), b.to(dev)], [wa.to(dev), wb.to(dev)], 1e-6), want, 3e-6)
    o, g = _rand(T, W, seed=5), _rand(T, W + 8, seed=6, scale=4.0)[:, 8:]
    _close(M.sigmoid_gate_mul(o.clone().to(dev), g.to(dev)), o.to(F64) * torch.sigmoid(g.to(F64)), 3e-6)
    y, z = _rand(T, W, seed=7), _rand(T, W, seed=8, scale=3.0)
    nw = _rand(W, seed=9) + 1.0
    parts = 2
    want = O.rms((y.to(F64) * O.silu(z.to(F64))).view(T, parts, W // parts), 1e-6).reshape(T, W) * nw.to(F64)
    got = M.gated_group_rms_norm(y.to(dev), nw.to(dev), z.to(dev), W // parts, 1e-6, torch.float32, gate_act="silu",
                                 gate_first=True)
    _close(got, want, 3e-6)


@pytest.mark.parametrize("tier", TIERS)
def test_gated_feed_forward(tier):
    dev = _dev(tier)
    layer = O.state_space_layer(mlp=O.dense(ff=56))
    hf = O.make_config([layer], width=48)
    W = O.random_weights(hf, seed=16)
    cfg = pogorax_config(hf)
    model = PogoraxForCausalLM(cfg)
    model.load_state_dict(convert_pogorax_state_dict(W, cfg), strict=False)
    mlp = model.to(dev).eval().model.layers[0].mlp
    h = _rand(21, 48, seed=17, scale=2.0)
    with torch.inference_mode():
        got = mlp(h.to(dev))
    _close(got, O.gated_ff(h.to(F64), O.to64(W), "l0.mlp."), 2e-5)
    assert math.isfinite(float(got.abs().max()))
