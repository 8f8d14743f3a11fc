"""The Domorax family served by the engine: random checkpoints in the family's file format, loaded by the framework's
loader and run through `LLMEngine.forward_ragged` / `generate` / the `replay` command, against the float64 oracle.
Covers whole prompts, token-by-token decoding, portions down to two tokens, batches of unequal requests, pages and state
slots that are given back and taken again, long decoding over many page borders and several windows, the first tokens,
and several layer orders and sizes (also sizes equal to one, and values that usual choices make equal)."""
import io
import json
import os

import numpy as np
import pytest
import torch

from colossalai_b200.inference.config import InferenceConfig
from colossalai_b200.inference.core.llm_engine import LLMEngine
from colossalai_b200.inference.struct import Sequence

from . import oracle as O

TIERS = ["plumbing", pytest.param("gpu", marks=pytest.mark.gpu)]

MODELS = {
    # every mixer once, a layer without feed-forward in the middle, dense and routed feed-forwards
    "mixed": dict(layers=[O.latent_layer(mlp="dense"), O.attention_layer(mlp="moe"), O.delta_layer(mlp=None),
                          O.latent_layer(heads=2, dim=16, rot_dim=4, vdim=8, kv_rank=12, q_rank=20, window=9, mlp="moe"),
                          O.attention_layer(heads=6, kv_heads=3, dim=8, conv=2, mlp="dense")]),
    # sizes that usual choices would hide: one head, one group, one expert, a window of one page and a half, a convolution
    # of one and of two taps, value heads wider than key heads, no stretched frequencies, no residual factor, one norm group
    "ones": dict(layers=[O.delta_layer(heads=1, kv_heads=1, dim=24, vdim=40, conv=2, mlp="dense"),
                         O.latent_layer(heads=1, dim=8, rot_dim=2, vdim=40, kv_rank=8, q_rank=8, window=12, scaling=None, mlp=None),
                         O.attention_layer(heads=1, kv_heads=1, dim=40, conv=1, mlp="moe"),
                         O.delta_layer(heads=5, kv_heads=5, dim=8, vdim=8, conv=3, mlp="moe")],
                 width=40, vocab=50, experts=1, top=1, shared_ff=0, groups=1, residual_mult=1.0),
    # attention only, in the other order; no window on one latent layer, a window longer than the prompts on the other;
    # every expert chosen; odd widths
    "attn": dict(layers=[O.attention_layer(heads=3, kv_heads=1, dim=24, conv=4, mlp="moe"),
                         O.latent_layer(heads=3, dim=24, rot_dim=6, vdim=10, kv_rank=20, q_rank=6, window=0, mlp="moe"),
                         O.latent_layer(heads=5, dim=6, rot_dim=10, vdim=6, kv_rank=14, q_rank=30, window=500,
                                        scaling=(8.0, 16, 2.0, 1.0), mlp="dense")],
                 width=30, experts=3, top=3, expert_ff=10, shared_ff=6, ff=21, groups=3, eps=1e-6, residual_mult=0.25),
    # rows wider than the tensor-core attention kernel takes (a latent row of 272 + 16 columns), heads of its widest row
    # (256), a delta rule with 256-wide keys, six taps, a window of one position, more experts than a warp has lanes
    "wide": dict(layers=[O.latent_layer(heads=2, dim=40, rot_dim=16, vdim=24, kv_rank=272, q_rank=24, window=40, mlp="moe"),
                         O.attention_layer(heads=2, kv_heads=1, dim=256, conv=6, mlp=None),
                         O.delta_layer(heads=2, kv_heads=1, dim=256, vdim=24, conv=6, mlp="dense"),
                         O.latent_layer(heads=3, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=8, window=1, mlp="moe")],
                 width=48, vocab=70, experts=33, top=5, expert_ff=8, shared_ff=8, ff=40, groups=6, eps=1e-5, residual_mult=0.5),
}


def _tier(tier):
    if tier == "gpu" and not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _engine(path, dtype=torch.float32, slots=3, pool_tokens=512, block_size=8, budget=4096, max_out=8, graphs=False):
    cfg = InferenceConfig(dtype=dtype, max_batch_size=slots, max_input_len=pool_tokens, max_output_len=max_out,
                          block_size=block_size, max_cache_tokens=pool_tokens, max_num_batched_tokens=budget,
                          use_cuda_graph=graphs)
    return LLMEngine(path, inference_config=cfg)


def _model(tmp_path, name, seed=0):
    kw = dict(MODELS[name])
    cfg = O.make_config(kw.pop("layers"), **kw)
    W = O.random_weights(cfg, seed=seed)
    return O.write_checkpoint(tmp_path / name, cfg, W), cfg, O.to64(W)


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _run(engine, schedule, prompts):
    """schedule: steps of [(request, n tokens)]; every position's logits are collected.  A request is admitted at its
    first entry and released after its last token."""
    handler = engine.request_handler
    at = {r: 0 for r in prompts}
    got = {r: [] for r in prompts}
    for step in schedule:
        entries, want = [], []
        for r, n in step:
            rs = handler.live.get(r) or handler.admit(Sequence(r, None, [], engine.inference_config.block_size, None,
                                                               -1, 0, max_output_len=1 << 30, ignore_eos=True))
            entries.append((rs, prompts[r][at[r]: at[r] + n]))
            want.append(list(range(n)))
            at[r] += n
        logits = engine.forward_ragged(entries, want).double().cpu()
        o = 0
        for r, n in step:
            got[r].append(logits[o:o + n])
            o += n
            if at[r] == len(prompts[r]):
                handler.release(r)
    return {r: torch.cat(v) for r, v in got.items()}


def _check(got, want, tol):
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    err = (d.pow(2).mean(-1).sqrt() / want.std()).max().item()
    assert err < tol, f"relative logit error {err:.3e}"


def _cuts(total, sizes):
    out, at = [], 0
    for n in sizes:
        n = min(n, total - at)
        if n > 0:
            out.append(n)
            at += n
    return out + [1] * (total - at)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("name", list(MODELS))
def test_whole_portions_and_decoding_agree_with_the_oracle(tmp_path, tier, name):
    _tier(tier)
    path, cfg, W = _model(tmp_path, name)
    L = 45
    toks = _tokens(L, cfg["vocab"], 1)
    want = O.forward(cfg, W, toks)
    eng = _engine(path)
    for sizes in ([L], [1] * L, [2, 2, 3, 7, 9, 2, 17], [8, 8, 8, 8], [7, 1, 1, 16, 2], [11, 1, 13, 2, 2, 2]):
        got = _run(eng, [[("a", n)] for n in _cuts(L, sizes)], {"a": toks})["a"]
        _check(got, want, 2e-4)
    assert eng.request_handler.cache_manager.num_available_blocks == eng.request_handler.cache_manager.total_num_blocks
    assert eng.request_handler.state_manager.num_available_slots == 3


@pytest.mark.parametrize("tier", TIERS)
def test_stream_after_every_layer(tmp_path, tier):
    _tier(tier)
    from colossalai_b200.models.hf_io import load_hf_checkpoint

    path, cfg, W = _model(tmp_path, "mixed", seed=2)
    dev = "cuda" if tier == "gpu" else "cpu"
    model = load_hf_checkpoint(path, dtype=torch.float32, device=dev).eval()
    toks = _tokens(17, cfg["vocab"], 3)
    want = []
    O.forward(cfg, W, toks, want)
    model.model.stream_trace = []
    with torch.inference_mode():
        model(input_ids=torch.tensor([toks], device=dev))
    assert len(model.model.stream_trace) == len(want) == 5
    for got, ref in zip(model.model.stream_trace, want):
        assert (got.double().cpu() - ref).abs().max() < 2e-4 * ref.abs().max()


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("name", list(MODELS))
def test_bfloat16_serving_stays_within_rounding(tmp_path, tier, name):
    """16-bit serving of every test model: also the widths that leave the kernels' vector paths."""
    _tier(tier)
    path, cfg, W = _model(tmp_path, name, seed=3)
    toks = _tokens(40, cfg["vocab"], 2)
    want = O.forward(cfg, W, toks)
    eng = _engine(path, dtype=torch.bfloat16)
    whole = _run(eng, [[("a", 40)]], {"a": toks})["a"]
    parts = _run(eng, [[("a", n)] for n in _cuts(40, [3, 2, 20])], {"a": toks})["a"]
    # per-head unit norms of read-outs that nearly cancel on the first tokens make single positions of these tiny models
    # sensitive to 16-bit rounding: the bound on the worst position is loose, the one on the average is not
    for got in (whole, parts):
        d = got - want
        d = d - d.mean(-1, keepdim=True)
        err = d.pow(2).mean(-1).sqrt() / want.std()
        assert err.max() < 0.2 and err.mean() < 3e-2, f"relative logit error: worst {err.max():.3e}, mean {err.mean():.3e}"


@pytest.mark.parametrize("tier", TIERS)
def test_mixed_batches_reuse_pages_and_slots(tmp_path, tier):
    """Five requests through two state slots and a pool of 14 pages: portions beside single tokens, a request that
    pauses, requests that end and whose pages and slot the next one takes."""
    _tier(tier)
    path, cfg, W = _model(tmp_path, "mixed", seed=5)
    lens = {"a": 50, "b": 1, "c": 23, "d": 37, "e": 9}
    prompts = {r: _tokens(n, cfg["vocab"], 20 + i) for i, (r, n) in enumerate(lens.items())}
    schedule = [[("b", 1), ("a", 10)],                                   # b ends at once: its slot goes to c
                [("a", 7), ("c", 2)], [("c", 1)], [("a", 2), ("c", 8)], [("a", 16), ("c", 1)],
                [("c", 11)],                                             # a pauses, c ends
                [("a", 1), ("d", 30)], [("a", 1), ("d", 1)], [("a", 13)],             # a ends
                [("d", 2), ("e", 2)], [("d", 1), ("e", 1)], [("d", 3), ("e", 6)]]      # e takes a's slot and pages
    eng = _engine(path, slots=2, pool_tokens=14 * 8, block_size=8)
    got = _run(eng, schedule, prompts)
    for r in prompts:
        _check(got[r], O.forward(cfg, W, prompts[r]), 2e-4)
    # the same request alone gives the same logits up to rounding
    alone = _run(_engine(path, slots=2, pool_tokens=14 * 8), [[("d", 37)]], {"d": prompts["d"]})["d"]
    _check(got["d"], alone, 1e-5)


@pytest.mark.parametrize("tier", TIERS)
def test_first_tokens_and_long_decoding(tmp_path, tier):
    _tier(tier)
    path, cfg, W = _model(tmp_path, "ones", seed=7)
    L = 150                                               # many page borders and twelve windows
    toks = _tokens(L, cfg["vocab"], 4)
    want = O.forward(cfg, W, toks)
    eng = _engine(path, block_size=16)
    got = _run(eng, [[("a", 1)]] + [[("a", 1)] for _ in range(L - 1)], {"a": toks})["a"]
    _check(got, want, 2e-4)
    got = _run(eng, [[("a", 2)], [("a", 1)], [("a", L - 3)]], {"a": toks})["a"]
    _check(got[:4], want[:4], 2e-4)
    _check(got, want, 2e-4)


@pytest.mark.parametrize("tier", TIERS)
def test_plain_forward_without_an_engine(tmp_path, tier):
    _tier(tier)
    from colossalai_b200.models.hf_io import load_hf_checkpoint

    path, cfg, W = _model(tmp_path, "attn", seed=9)
    dev = "cuda" if tier == "gpu" else "cpu"
    model = load_hf_checkpoint(path, dtype=torch.float32, device=dev).eval()
    a, b = _tokens(19, cfg["vocab"], 1), _tokens(19, cfg["vocab"], 2)
    with torch.inference_mode():
        out = model(input_ids=torch.tensor([a, b], device=dev))["logits"].double().cpu().view(2, 19, -1)
    _check(out[0], O.forward(cfg, W, a), 2e-4)
    _check(out[1], O.forward(cfg, W, b), 2e-4)


@pytest.mark.parametrize("tier", TIERS)
def test_greedy_generation_through_the_scheduler(tmp_path, tier):
    """`generate` on more requests than slots, with a token budget that cuts prompts into portions."""
    _tier(tier)
    path, cfg, W = _model(tmp_path, "mixed", seed=11)
    prompts = [_tokens(n, cfg["vocab"], 30 + n) for n in (21, 3, 34, 9)]
    new = 6
    eng = _engine(path, slots=2, pool_tokens=256, budget=16, max_out=new)
    eng.inference_config.ignore_eos = True
    _, ids = eng.generate(prompts_token_ids=[list(p) for p in prompts], return_token_ids=True)
    for p, full in zip(prompts, ids):
        seq = list(p)
        for _ in range(new):
            logits = O.forward(cfg, W, seq)[-1]
            top = torch.topk(logits, 2).values
            if top[0] - top[1] < 1e-3 * logits.std():      # a near tie may resolve either way in fp32
                seq.append(full[len(seq)])
                continue
            seq.append(int(logits.argmax()))
        assert full == seq
    assert eng.request_handler.state_manager.num_available_slots == 2


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["mixed", "ones"])
def test_graph_replayed_decode_steps_match_eager_ones(tmp_path, name):
    """Decode steps replayed from CUDA graphs (fixed layout buffer, worst-case launch shapes) against eager steps:
    three sequences of unequal length decode side by side, one ends early so the batch size changes."""
    _tier("gpu")
    path, cfg, W = _model(tmp_path, name, seed=17)
    lens = {"a": 70, "b": 9, "c": 33}
    prompts = {r: _tokens(n, cfg["vocab"], 40 + i) for i, (r, n) in enumerate(lens.items())}
    schedule = [[("a", 40), ("b", 3), ("c", 20)]] + [[("a", 1), ("b", 1), ("c", 1)]] * 6 + \
        [[("a", 1), ("c", 1)]] * 7 + [[("a", 1)]] * 17
    eager = _run(_engine(path, dtype=torch.bfloat16, block_size=16), schedule, prompts)
    eng = _engine(path, dtype=torch.bfloat16, block_size=16, graphs=True)
    assert sorted(eng.ragged_graphs) == [1, 2]            # the ladder of batch sizes up to three slots
    replayed = _run(eng, schedule, prompts)
    for r in prompts:
        _check(replayed[r], eager[r], 3e-2)


@pytest.mark.parametrize("tier", TIERS)
def test_replay_command_writes_the_logits_asked_for(tmp_path, tier):
    _tier(tier)
    from colossalai_b200.cli.replay import replay

    path, cfg, W = _model(tmp_path, "attn", seed=13)
    a, b = _tokens(20, cfg["vocab"], 5), _tokens(6, cfg["vocab"], 6)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:12], "want": [0, 11]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[12:13], "want": []}, {"id": "b", "tokens": b, "want": [5]}],
              "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[13:], "want": [6]}], "end": ["a"]}]
    out, answers = tmp_path / "out", io.StringIO()
    rc = replay(path, "float32", str(out), 64, io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), answers)
    assert rc == 0 and answers.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    wa, wb = O.forward(cfg, W, a), O.forward(cfg, W, b)
    g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)).double()
    g1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)).double()
    g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1)).double()
    _check(g0, wa[[0, 11]], 2e-4)
    _check(g1, wb[[5]], 2e-4)
    _check(g2, wa[[19]], 2e-4)
    assert sorted(os.listdir(out)) == ["0.f32", "1.f32", "2.f32"]
