"""Serving throughput of a hybrid decoder (Gopunex layers: channel-wise delta rule / bias+sink attention / lightning
attention) beside a Llama of equal width, depth and head sizes, both with random weights through `LLMEngine`, plus the
time of every mixer kernel alone against its roofline.  `--family palilix` runs the Palilix family (parallel layers with
retention / latent attention, dense and routed feed-forwards, a looped span) beside Gopunex, the closest served family,
at equal width and number of layer runs, and its kernels beside their like kernels; `--family pogorax` does the same
for the Pogorax family (pairs of attention and a recurrent mixer side by side, selective state spaces, pre-norm layers),
`--family domorax` for the Domorax family (windowed latent attention with sinks, convolved attention with distance slopes,
delta rule with a decay per head, grouped output norms, a depth-weighted stream, normalised-power and routed feed-forwards).

    python examples/inference/benchmark_hybrid.py [--sizes 2048x8,4096x4] [--batch 8] [--in_len 2048] [--out_len 64]
                                                  [--family gopunex|palilix|pogorax|domorax]

Also reachable as `python bench.py --workload hybrid-serve`.  One JSON line per (size, family) and one per kernel.
Timing: CUDA events on the launching stream after warm-up; the kernel timings write a 256 MB buffer between runs (L2
flush).  Rooflines use the measured copy bandwidth / bf16 GEMM throughput of MEASURED_PEAKS.json.
"""
import argparse
import gc
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from colossalai_b200.inference import GenerationConfig, InferenceConfig  # noqa: E402
from colossalai_b200.inference.core.llm_engine import LLMEngine  # noqa: E402
from colossalai_b200.models import build_model  # noqa: E402
from colossalai_b200.models.config import ExpertFFSpec, LayerSpec, MixerSpec, ModelConfig  # noqa: E402

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..")


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return p["hbm_gbs"] * 1e9, p["bf16_tflops"] * 1e12, "measured"
    except Exception:
        return 6.65e12, 1.59e15, "fallback"


def hybrid_config(width: int, layers: int, vocab: int = 32000) -> ModelConfig:
    H, d = width // 128, 128
    att = MixerSpec(kind="attention", heads=H, kv_heads=max(H // 4, 1), dim=d, vdim=d, bias=True, scale=d ** -0.5,
                    bias_buckets=32, bias_max=512.0, sink=True, proj_norm=True, v_mix=True)
    lig = MixerSpec(kind="lightning", heads=H, dim=d, vdim=d, decay=[1.0 - 2.0 ** -(5 + 3 * i / H) for i in range(H)])
    dlt = MixerSpec(kind="channel_delta", heads=H, kv_heads=H, dim=d, vdim=d, conv=4, decay_rank=64, gate_rank=64)
    order = [dlt, att, lig, dlt, att]
    specs = [LayerSpec(mixer=order[i % len(order)], ff=4 * width) for i in range(layers)]
    return ModelConfig(model_type="gopunex", vocab_size=vocab, hidden_size=width, intermediate_size=4 * width,
                       layer_specs=specs, norm_eps=1e-5, hidden_act="relu2", glu=False, pos_type="none",
                       norm_placement="sublayer_out", residual_mult=0.7, norm_weight_offset=1.0, fp32_residual=True,
                       max_position_embeddings=1 << 20)


def palilix_config(width: int, runs: int, vocab: int = 32000, kv_rank: int = 192, rot: int = 64) -> ModelConfig:
    """`runs` layer runs: runs - 2 distinct layers of which the second and third run twice.  Heads of 128 channels;
    latent rows of kv_rank + rot = 256 columns; every other layer has routed experts (8, top 2) with a shared expert."""
    H, d = width // 128, 128
    ret = MixerSpec(kind="retention", heads=H, dim=d, vdim=d, decay=[1.0 - 2.0 ** -(5 + 3 * i / H) for i in range(H)],
                    rot_dims=64, rot_base=1e6)
    lat = MixerSpec(kind="latent", heads=H, kv_heads=1, dim=d - rot, rot_dim=rot, rot_dims=rot, vdim=d, kv_rank=kv_rank,
                    rot_base=5e5, scale=d ** -0.5)
    moe = ExpertFFSpec(experts=8, top=2, ff=width, limit=7.0, shared_ff=2 * width, shared_limit=7.0)
    order = [(ret, None), (ret, moe), (lat, moe), (lat, None)]
    n = max(runs - 2, 3)
    specs = [LayerSpec(mixer=order[i % 4][0], ff=None if order[i % 4][1] else 4 * width, moe=order[i % 4][1])
             for i in range(n)]
    return ModelConfig(model_type="palilix", vocab_size=vocab, hidden_size=width, intermediate_size=4 * width,
                       layer_specs=specs, norm_eps=1e-5, norm_type="layer", norm_bias=False, hidden_act="gelu_tanh",
                       glu=False, pos_type="none", parallel_block=True, fp32_residual=True, embed_scale=1.0,
                       logit_scale=1.0, logit_softcap=30.0, loop_start=1, loop_stop=3, loop_times=2,
                       max_position_embeddings=1 << 20)


def pogorax_config(width: int, layers: int, vocab: int = 32000) -> ModelConfig:
    """Layers [rotary attention | linear recurrent unit, gated block-masked attention | matrix memory, state space, ...]:
    attention heads of 128 (one key / value head per four query heads), rotary positions on half of every head, mask blocks
    of 1024 positions; a recurrent unit as wide as the model with gate blocks of 128; matrix-memory heads of 64 x 128;
    state-space heads of 64 channels with 128 state rows over twice the model width; gated feed-forwards of 8/3 x width
    (none behind the state space)."""
    H, d = width // 128, 128
    G = max(H // 4, 1)
    rot = MixerSpec(kind="attention", heads=H, kv_heads=G, dim=d, vdim=d, scale=d ** -0.5, rot_dims=64, rot_base=5e5,
                    rot_interleaved=True, head_unit_norm=True, wide_weights=True)
    lru = MixerSpec(kind="rglru", lru_width=width, blocks=H, conv=4)
    gat = MixerSpec(kind="attention", heads=H, kv_heads=G, dim=d, vdim=d, scale=d ** -0.5, mask_block=1024, out_gate=True,
                    wide_weights=True)
    mem = MixerSpec(kind="mlstm", heads=H, dim=64, vdim=d, gate_cap=15.0)
    ssd = MixerSpec(kind="ssd", heads=2 * width // 64, vdim=64, dim=128, state=128, groups=1, norm_groups=1, conv=4)
    ff = width * 8 // 3 // 64 * 64
    order = [(MixerSpec(kind="pair", parts=[rot, lru]), ff), (MixerSpec(kind="pair", parts=[gat, mem]), ff), (ssd, None)]
    specs = [LayerSpec(mixer=order[i % 3][0], ff=order[i % 3][1]) for i in range(layers)]
    return ModelConfig(model_type="pogorax", vocab_size=vocab, hidden_size=width, intermediate_size=ff, layer_specs=specs,
                       norm_eps=1e-6, norm_type="rms", hidden_act="gelu_tanh", glu=True, pos_type="none", embed_scale=1.0,
                       fp32_residual=True, fp32_logits=True, max_position_embeddings=1 << 20)


def domorax_config(width: int, layers: int, vocab: int = 32000, kv_rank: int = 192, rot: int = 64) -> ModelConfig:
    """Layers [latent attention + dense, convolved attention + routed, delta rule + routed, latent attention + routed, ...].
    Heads of 128 channels.  Latent attention: queries through a latent of 3/8 of the width, cache rows of kv_rank + rot = 256
    columns, a window of 1024 positions, learned sinks, frequencies stretched by 4 beyond 4096 positions.  Convolved
    attention: one key head per four query heads, four taps.  Delta rule: one q / k head per two value heads, four taps.
    Dense feed-forwards of 4 x width, eight experts of 1 x width (top 2) with a gated shared expert of 2 x width; output
    norms in 4 groups, residual factor 0.5."""
    H, d = width // 128, 128
    lat = MixerSpec(kind="latent", heads=H, kv_heads=1, dim=d - rot, rot_dim=rot, rot_dims=rot, vdim=d, kv_rank=kv_rank,
                    rot_base=5e5, scale=d ** -0.5, q_rank=width * 3 // 8, window=1024, sink_learned=True,
                    rot_scaling=[4.0, 4096.0, 32.0, 1.0], wide_weights=True)
    att = MixerSpec(kind="attention", heads=H, kv_heads=max(H // 4, 1), dim=d, vdim=d, scale=d ** -0.5, conv=4,
                    head_norm=True, values_from_keys=True, dist_slopes=True, wide_weights=True)
    dlt = MixerSpec(kind="delta", heads=H, kv_heads=max(H // 2, 1), dim=d, vdim=d, conv=4)
    moe = ExpertFFSpec(experts=8, top=2, ff=width, act="silu", shared_ff=2 * width, shared_gate=True)
    order = [(lat, None), (att, moe), (dlt, moe), (lat, moe)]
    specs = [LayerSpec(mixer=order[i % 4][0], ff=None if order[i % 4][1] else 4 * width, moe=order[i % 4][1],
                       ff_act=None if order[i % 4][1] else "polynorm") for i in range(layers)]
    return ModelConfig(model_type="domorax", vocab_size=vocab, hidden_size=width, intermediate_size=4 * width,
                       layer_specs=specs, norm_eps=1e-5, norm_groups=4, norm_type="rms", hidden_act="polynorm", glu=False,
                       pos_type="none", norm_placement="sublayer_out", residual_mult=0.5, fp32_residual=True,
                       depth_average=True, fp32_logits=True, max_position_embeddings=1 << 20)


def llama_config(width: int, layers: int, vocab: int = 32000) -> ModelConfig:
    H = width // 128
    # 8/3 x width gated feed-forward = the parameter count of the hybrid's 4 x width plain one
    return ModelConfig(model_type="llama", vocab_size=vocab, hidden_size=width, intermediate_size=width * 8 // 3 // 64 * 64,
                       num_hidden_layers=layers, num_attention_heads=H, num_key_value_heads=max(H // 4, 1), head_dim=128,
                       max_position_embeddings=1 << 16)


def build(cfg: ModelConfig):
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = build_model(cfg).to(torch.bfloat16)
    with torch.no_grad():
        for n, p in model.named_parameters():          # recurrent layers: non-degenerate convolutions and decays
            if n.endswith("conv_weight"):
                p.normal_(0, 0.5)
            elif n.endswith("dt_bias") or n.endswith("rel_bias"):
                p.normal_(0, 1.0)
            elif n.endswith("v_mix"):
                p.fill_(0.4)
            elif n.endswith("act_coef"):
                p.copy_(torch.tensor([0.6, 0.3, 0.1, 0.0]))
            elif n.endswith("depth_weight"):
                p.fill_(1.0 / p.numel())
    return model.eval()


def serve(cfg: ModelConfig, batch: int, in_len: int, out_len: int, cuda_graph: bool = False) -> dict:
    model = build(cfg)
    icfg = InferenceConfig(max_batch_size=batch, max_input_len=in_len, max_output_len=out_len, dtype="bf16",
                           block_size=64, ignore_eos=True, max_num_batched_tokens=batch * in_len,
                           use_cuda_graph=cuda_graph)
    eng = LLMEngine(model, None, icfg)
    gen = GenerationConfig(max_new_tokens=out_len)
    eng.generation_config, eng.generation_config_dict = gen, gen.to_dict()
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(3, cfg.vocab_size, (batch, in_len), generator=g).tolist()

    def run():
        eng.add_request(prompts_token_ids=prompts, generation_config=gen)
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        eng.step()
        e1.record()
        steps = 0
        while eng.request_handler.check_unfinished_reqs():
            eng.step()
            steps += 1
        e2.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), e1.elapsed_time(e2), steps

    run()
    run()
    from colossalai_b200.kernel import loader

    loader.launch_counter.reset()
    tp, td, steps = run()
    n_params = sum(p.numel() for p in model.parameters())
    out = {"family": cfg.model_type, "width": cfg.hidden_size, "layers": cfg.num_hidden_layers, "params": n_params,
           "layer_runs": cfg.num_cache_layers, "batch": batch, "in_len": in_len, "out_len": out_len, "cuda_graph": cuda_graph, "prefill_ms": tp,
           "prefill_tokens_per_s": batch * in_len / (tp / 1e3), "decode_ms_per_step": td / max(steps, 1),
           "decode_tokens_per_s": batch * steps / (td / 1e3), "our_kernel_launches": loader.launch_counter.count}
    del eng, model, run
    gc.collect()                                # graphs of this engine go now, not in the middle of the next capture
    torch.cuda.empty_cache()
    return out


def _time(fn, flush, iters: int = 5, graph: bool = False) -> float:
    """Median device time of `fn`.  `graph`: the launches are captured once and replayed, which takes the host's share
    (python and launch latency, tens of microseconds) out of kernels that run for a few microseconds."""
    for _ in range(3):
        fn()
    if graph:
        g = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            fn()
        fn = g.replay
        fn()
    ts = []
    for _ in range(iters):
        flush.add_(1)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return sorted(ts)[len(ts) // 2]


def kernels(width: int, batch: int, in_len: int) -> list:
    """Every mixer kernel alone at one layer's sizes, prefill (batch x in_len tokens) and decode (batch tokens on
    in_len of context), beside Llama's flash prefill and paged decode attention."""
    from colossalai_b200 import ops
    from colossalai_b200.ops import inference as iops
    from colossalai_b200.ops import mixers as M

    hbm, tflops, src = peaks()
    dev, dt = "cuda", torch.bfloat16
    H, d, G, bs = width // 128, 128, max(width // 128 // 4, 1), 64
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    rows = []

    def rec(name, phase, ms, bytes_, flops, like=""):
        ideal = max(bytes_ / hbm, flops / tflops) * 1e3
        rows.append({"kernel": name, "phase": phase, "width": width, "ms": ms, "roofline_ms": ideal,
                     "frac_of_" + src + "_roofline": ideal / ms, "bound": "hbm" if bytes_ / hbm > flops / tflops else "tensor",
                     "like": like})

    for phase, q_len, ctx in (("prefill", in_len, 0), ("decode", 1, in_len)):
        T = batch * q_len
        meta = M.RaggedMeta.build([q_len] * batch, [ctx] * batch, list(range(batch)), dev)
        x = lambda c: torch.randn(T, c, device=dev, dtype=dt)
        S = torch.zeros(batch, H, d, d, device=dev)
        state_bytes = 2 * S.numel() * 4
        q, k, v, a, b = x(H * d) * 0.1, x(H * d) * 0.1, x(H * d), x(H * d), x(H)
        al, db = torch.zeros(H, device=dev), torch.zeros(H * d, device=dev)
        ms = _time(lambda: M.state_scan_delta(q, k, v, a, b, al, db, S, meta, H, H, d, d), flush)
        rec("state_scan_delta", phase, ms, T * (4 * H * d * 2 + H * d * 4) + state_bytes, 6.0 * T * H * d * d)
        dec = torch.full((H,), 0.97, device=dev)
        ms = _time(lambda: M.state_scan_decay(q, k, v, dec, S, meta, H, d, d), flush)
        rec("state_scan_decay", phase, ms, T * (3 * H * d * 2 + H * d * 4) + state_bytes, 4.0 * T * H * d * d)
        C = 3 * H * d
        xc, w, st = x(C), torch.randn(C, 4, device=dev, dtype=dt), torch.zeros(batch, 3, C, device=dev, dtype=dt)
        ms = _time(lambda: M.short_conv_silu(xc, w, st, meta), flush)
        rec("short_conv_silu", phase, ms, 2 * T * C * 2, 0)
        o, gate, wn = torch.randn(T, H * d, device=dev), x(H * d), torch.ones(d, device=dev, dtype=dt)
        ms = _time(lambda: M.gated_group_rms_norm(o, wn, gate, d, 1e-5, dt), flush)
        rec("gated_group_rmsnorm", phase, ms, T * H * d * (4 + 2 + 2), 0)
        xs, y, wr = torch.randn(T, width, device=dev), x(width), torch.zeros(width, device=dev, dtype=dt)
        ms = _time(lambda: M.rms_norm_residual(xs, y, wr, 1e-5, 0.7, 1.0), flush)
        rec("rmsnorm_residual", phase, ms, T * width * (4 + 4 + 2 + 2), 0, like="rmsnorm_fwd(+residual)")
        yl, wl = x(width), torch.ones(width, device=dev, dtype=dt)
        ms = _time(lambda: ops.rms_norm(yl, wl, 1e-5, yl), flush)
        rec("llama:rmsnorm_fwd(+residual)", phase, ms, T * width * 2 * 4, 0)
        # attention over pages: ours (bias + sink, ragged) and Llama's (flash prefill / split-KV decode)
        L = ctx + q_len
        per = (L + bs - 1) // bs
        kc = torch.randn(batch * per, bs, G, d, device=dev, dtype=dt)
        vc = torch.randn(batch * per, bs, G, d, device=dev, dtype=dt)
        tables = torch.arange(batch * per, dtype=torch.int32, device=dev).view(batch, per)
        qa = x(H * d)
        rel = torch.randn(32, H, device=dev)
        starts_host = M.log_bucket_starts(32, 512.0)
        starts = torch.tensor(starts_host, dtype=torch.int32, device=dev)
        lut = M.bucket_lut(starts_host).to(dev)               # built once per layer by the model as well
        ms = _time(lambda: M.paged_bias_attention(qa, kc, vc, tables, meta, d ** -0.5, rel, starts, True, lut=lut),
                   flush)
        kv_bytes = 2 * batch * L * G * d * 2
        att_flops = 4.0 * batch * H * d * (q_len * ctx + q_len * (q_len + 1) / 2)
        rec("paged_bias_attention", phase, ms, kv_bytes + 2 * T * H * d * 2, att_flops,
            like="flash prefill" if phase == "prefill" else "paged decode")
        if phase == "prefill":
            q3, k3, v3 = qa.view(T, H, d), x(G * d).view(T, G, d), x(G * d).view(T, G, d)
            cu = torch.arange(0, T + 1, q_len, dtype=torch.int32, device=dev)
            ms = _time(lambda: ops.attention(q3, k3, v3, causal=True, scale=d ** -0.5, cu_seqlens_q=cu, cu_seqlens_k=cu,
                                             max_seqlen=q_len), flush)
            rec("llama:flash_prefill_attention", phase, ms, kv_bytes + 2 * T * H * d * 2, att_flops)
        else:
            lens = torch.full((batch,), L, dtype=torch.int32, device=dev)
            ms = _time(lambda: iops.paged_decode_attention(qa.view(T, H, d), kc, vc, tables, lens, d ** -0.5), flush)
            rec("llama:paged_decode_attention", phase, ms, kv_bytes + 2 * T * H * d * 2, att_flops)
    return rows


def kernels_palilix(width: int, batch: int, in_len: int, kv_rank: int = 192, rot: int = 64) -> list:
    """Every kernel of the Palilix layers alone at one layer's sizes beside its like kernel of the closest families."""
    from colossalai_b200 import ops
    from colossalai_b200.ops import inference as iops
    from colossalai_b200.ops import mixers as M
    from colossalai_b200.ops.moe import gather_combine

    hbm, tflops, src = peaks()
    dev, dt = "cuda", torch.bfloat16
    H, d, bs = width // 128, 128, 64
    G = max(H // 4, 1)
    Dk = kv_rank + rot
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    rows = []

    def rec(name, phase, ms, bytes_, flops, like=""):
        ideal = max(bytes_ / hbm, flops / tflops) * 1e3
        rows.append({"kernel": name, "phase": phase + ("(graph replay)" if phase == "decode" else ""), "width": width, "ms": ms, "roofline_ms": ideal,
                     "frac_of_" + src + "_roofline": ideal / ms, "bound": "hbm" if bytes_ / hbm > flops / tflops else "tensor",
                     "like": like})

    for phase, q_len, ctx in (("prefill", in_len, 0), ("decode", 1, in_len)):
        replay = phase == "decode"             # decode kernels are timed as graph replays (no host share)
        T = batch * q_len
        meta = M.RaggedMeta.build([q_len] * batch, [ctx] * batch, list(range(batch)), dev)
        x = lambda c: torch.randn(T, c, device=dev, dtype=dt)
        # stream sum + layer norm  |  like: Gopunex norm + residual, Llama fused norm
        xs, y1, y2 = torch.randn(T, width, device=dev), x(width), x(width)
        w = torch.ones(width, device=dev, dtype=dt)
        ms = _time(lambda: M.stream_add_norm(xs, [y1, y2], weight=w, eps=1e-5, kind="layer"), flush, graph=replay)
        rec("stream_add_norm(2 addends, layer norm)", phase, ms, T * width * (4 + 4 + 2 + 2 + 2), 0, like="rmsnorm_residual")
        ms = _time(lambda: M.rms_norm_residual(xs, y1, w, 1e-5, 0.7, 1.0), flush, graph=replay)
        rec("gopunex:rmsnorm_residual", phase, ms, T * width * (4 + 4 + 2 + 2), 0)
        ms = _time(lambda: ops.rms_norm(y1, w, 1e-5, y2), flush, graph=replay)
        rec("llama:rmsnorm_fwd(+residual)", phase, ms, T * width * 2 * 4, 0)
        # retention scan with rotary positions  |  like: the same scan without them (lightning attention)
        S = torch.zeros(batch, H, d, d, device=dev)
        state_bytes = 2 * S.numel() * 4
        q, k, v = x(H * d) * 0.1, x(H * d) * 0.1, x(H * d)
        dec = torch.full((H,), 0.97, device=dev)
        table = M.rotary_table(ctx + q_len, 64, 1e6, dev)
        ms = _time(lambda: M.state_scan_decay(q, k, v, dec, S, meta, H, d, d, act_silu=False, rot_table=table, rot_dims=64,
                                              k_scale=d ** -0.5), flush, graph=replay)
        rec("state_scan_decay+rotary", phase, ms, T * (3 * H * d * 2 + H * d * 4) + state_bytes, 4.0 * T * H * d * d,
            like="state_scan_decay")
        ms = _time(lambda: M.state_scan_decay(q, k, v, dec, S, meta, H, d, d), flush, graph=replay)
        rec("gopunex:state_scan_decay", phase, ms, T * (3 * H * d * 2 + H * d * 4) + state_bytes, 4.0 * T * H * d * d)
        o, gate, wn = torch.randn(T, H * d, device=dev), x(H * d), torch.ones(d, device=dev, dtype=dt)
        ms = _time(lambda: M.gated_group_rms_norm(o, None, gate, d, 1e-5, dt, gate_act="silu"), flush, graph=replay)
        rec("gated_group_rmsnorm(silu)", phase, ms, T * H * d * (4 + 2 + 2), 0, like="gated_group_rmsnorm")
        ms = _time(lambda: M.gated_group_rms_norm(o, wn, gate, d, 1e-5, dt), flush, graph=replay)
        rec("gopunex:gated_group_rmsnorm", phase, ms, T * H * d * (4 + 2 + 2), 0)
        # latent attention: cache rows, query rotation, attention over the rows
        L = ctx + q_len
        per = (L + bs - 1) // bs
        cache = torch.randn(batch * per, bs, 1, Dk, device=dev, dtype=dt)
        tables = torch.arange(batch * per, dtype=torch.int32, device=dev).view(batch, per)
        z, nw = x(Dk), torch.ones(kv_rank, device=dev, dtype=dt)
        tab_r = M.rotary_table(L, rot, 5e5, dev)
        ms = _time(lambda: M.latent_kv_write(z, nw, 1e-5, kv_rank, tab_r, cache, tables, meta), flush, graph=replay)
        rec("latent_kv_write", phase, ms, 2 * T * Dk * 2, 0, like="paged_kv_write_mix")
        kc = torch.randn(batch * per, bs, G, d, device=dev, dtype=dt)
        vc = torch.randn(batch * per, bs, G, d, device=dev, dtype=dt)
        kk, vv = x(G * d), x(G * d)
        ms = _time(lambda: M.paged_kv_write_mix(kk, vv, kc, vc, tables, meta), flush, graph=replay)
        rec("gopunex:paged_kv_write_mix", phase, ms, 2 * T * 2 * G * d * 2, 0)
        qs, qa = x(H * d), torch.empty(T, H * Dk, device=dev, dtype=dt)
        ms = _time(lambda: M.rotary_half(qs, qa, H, d, d - rot, Dk, kv_rank, rot, rot, tab_r, meta.token_pos), flush, graph=replay)
        rec("rotary_half(q part)", phase, ms, 2 * T * H * rot * 2, 0, like="rope_qkv")
        qkv = x(H * d)                                      # Llama's in-place rotation of the same number of channels
        cos, sin = ops.build_rope_cache(L, rot, 5e5, device=dev)
        posl = meta.token_pos.long()
        ms = _time(lambda: ops.rope_qkv(qkv, posl, cos, sin, H, 0, d, rot_dim=rot), flush, graph=replay)
        rec("llama:rope_qkv", phase, ms, 2 * T * H * rot * 2, 0)
        qa.normal_()
        ms = _time(lambda: M.paged_bias_attention(qa, cache, cache, tables, meta, d ** -0.5, vdim=kv_rank), flush, graph=replay)
        kv_bytes = batch * L * Dk * 2
        att_flops = 2.0 * batch * H * (Dk + kv_rank) * (q_len * ctx + q_len * (q_len + 1) / 2)
        rec("latent_attention", phase, ms, kv_bytes + T * H * (Dk + kv_rank) * 2, att_flops,
            like="paged_bias_attention")
        qg = x(H * d)
        rel = torch.randn(32, H, device=dev)
        starts_host = M.log_bucket_starts(32, 512.0)
        starts = torch.tensor(starts_host, dtype=torch.int32, device=dev)
        lut = M.bucket_lut(starts_host).to(dev)
        ms = _time(lambda: M.paged_bias_attention(qg, kc, vc, tables, meta, d ** -0.5, rel, starts, True, lut=lut), flush, graph=replay)
        g_bytes = 2 * batch * L * G * d * 2 + 2 * T * H * d * 2
        g_flops = 4.0 * batch * H * d * (q_len * ctx + q_len * (q_len + 1) / 2)
        rec("gopunex:paged_bias_attention", phase, ms, g_bytes, g_flops)
        if phase == "decode":
            lens = torch.full((batch,), L, dtype=torch.int32, device=dev)
            ms = _time(lambda: iops.paged_decode_attention(qg.view(T, H, d), kc, vc, tables, lens, d ** -0.5), flush, graph=replay)
            rec("llama:paged_decode_attention", phase, ms, g_bytes, g_flops)
        # experts: clamped gated unit (top 2 of every token), fp32 gather-combine
        I = width
        gu = x(2 * I).repeat(2, 1)
        ms = _time(lambda: ops.clamped_glu(gu, 7.0, 1.702), flush, graph=replay)
        rec("clamped_glu", phase, ms, 2 * T * 3 * I * 2, 0, like="glu_fwd(silu)")
        ms = _time(lambda: ops.glu(gu, "silu"), flush, graph=replay)
        rec("llama:glu_fwd(silu)", phase, ms, 2 * T * 3 * I * 2, 0)
        ys = x(width).repeat(2, 1)
        row_of = torch.randperm(2 * T, device=dev).view(T, 2)
        wts = torch.rand(T, 2, device=dev)
        ms = _time(lambda: gather_combine(ys, row_of, wts), flush, graph=replay)
        rec("moe_gather_combine", phase, ms, T * width * (2 * 2 + 4), 0)
    return rows


def kernels_pogorax(width: int, batch: int, in_len: int) -> list:
    """Every kernel of the Pogorax layers alone at one layer's sizes beside its like kernel of the closest families."""
    from colossalai_b200 import ops
    from colossalai_b200.ops import mixers as M

    hbm, tflops, src = peaks()
    dev, dt = "cuda", torch.bfloat16
    H, d, bs = width // 128, 128, 64
    G = max(H // 4, 1)
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    rows = []

    def rec(name, phase, ms, bytes_, flops, like=""):
        ideal = max(bytes_ / hbm, flops / tflops) * 1e3
        rows.append({"kernel": name, "phase": phase + ("(graph replay)" if phase == "decode" else ""), "width": width, "ms": ms, "roofline_ms": ideal,
                     "frac_of_" + src + "_roofline": ideal / ms, "bound": "hbm" if bytes_ / hbm > flops / tflops else "tensor",
                     "like": like})

    for phase, q_len, ctx in (("prefill", in_len, 0), ("decode", 1, in_len)):
        replay = phase == "decode"             # decode kernels are timed as graph replays (no host share)
        T = batch * q_len
        meta = M.RaggedMeta.build([q_len] * batch, [ctx] * batch, list(range(batch)), dev)
        x = lambda c: torch.randn(T, c, device=dev, dtype=dt)
        # stream sum + RMS norm, mean of two normed mixer outputs  |  like: Gopunex norm + residual
        xs, y1, y2 = torch.randn(T, width, device=dev), x(width), x(width)
        w = torch.ones(width, device=dev, dtype=dt)
        ms = _time(lambda: M.stream_add_norm(xs, [y1], weight=w, eps=1e-6, kind="rms"), flush, graph=replay)
        rec("stream_add_norm(1 addend, rms)", phase, ms, T * width * (4 + 4 + 2 + 2), 0, like="rmsnorm_residual")
        ms = _time(lambda: M.norm_mean([y1, y2], [w, w], 1e-6), flush, graph=replay)
        rec("norm_mean(2 parts)", phase, ms, T * width * (2 + 2 + 4), 0, like="rmsnorm_residual")
        ms = _time(lambda: M.rms_norm_residual(xs, y1, w, 1e-5, 0.7, 1.0), flush, graph=replay)
        rec("gopunex:rmsnorm_residual", phase, ms, T * width * (4 + 4 + 2 + 2), 0)
        # matrix memory (heads of 64 x 128), state space (width / 32 heads of 128 x 64)  |  like: the decay scan
        Hm, dm = H, 64
        S = torch.zeros(batch, Hm, dm, d, device=dev)
        n_, m_ = torch.zeros(batch, Hm, dm, device=dev), torch.zeros(batch, Hm, device=dev)
        q, k, v, gates = x(Hm * dm) * 0.1, x(Hm * dm) * 0.1, x(Hm * d), x(2 * Hm)
        gb = torch.zeros(2 * Hm, device=dev)
        ms = _time(lambda: M.state_scan_mlstm(q, k, v, gates, gb, 15.0, S, n_, m_, meta, Hm, dm, d, dm ** -0.5), flush,
                   graph=replay)
        rec("state_scan_mlstm", phase, ms, T * (2 * Hm * dm * 2 + Hm * d * 2 + Hm * d * 4) + 2 * S.numel() * 4,
            4.0 * T * Hm * dm * d, like="state_scan_decay")
        Hs, N, dv = 2 * width // 64, 128, 64
        Ss = torch.zeros(batch, Hs, N, dv, device=dev)
        c_, b_, xs_, dtr = x(N), x(N), x(Hs * dv), x(Hs)
        z3 = torch.zeros(Hs, device=dev)
        ms = _time(lambda: M.state_scan_ssd(c_, b_, xs_, dtr, z3, z3, z3, Ss, meta, Hs, 1, N, dv), flush, graph=replay)
        rec("state_scan_ssd", phase, ms, T * (2 * N * 2 + Hs * dv * 2 + Hs * dv * 4) + 2 * Ss.numel() * 4,
            4.0 * T * Hs * N * dv, like="state_scan_decay")
        Sg = torch.zeros(batch, H, d, d, device=dev)
        qg, kg, vg = x(H * d) * 0.1, x(H * d) * 0.1, x(H * d)
        dec = torch.full((H,), 0.97, device=dev)
        ms = _time(lambda: M.state_scan_decay(qg, kg, vg, dec, Sg, meta, H, d, d), flush, graph=replay)
        rec("gopunex:state_scan_decay", phase, ms, T * (3 * H * d * 2 + H * d * 4) + 2 * Sg.numel() * 4, 4.0 * T * H * d * d)
        # linear recurrent unit: one thread per channel  |  like: the convolution (the other per-channel walk over time)
        C = width
        u, br = x(C), x(C)
        gts = torch.randn(H, T, 2 * C // H, device=dev)
        gbi, lam, Sl = torch.zeros(H, 2 * C // H, device=dev), torch.zeros(C, device=dev), torch.zeros(batch, C, device=dev)
        ms = _time(lambda: M.lru_scan(u, gts, gbi, lam, br, Sl, meta), flush, graph=replay)
        rec("lru_scan", phase, ms, T * C * (8 + 2 + 2 + 2), 0, like="short_conv_silu")
        Cc = 2 * width + 2 * N
        xc, wc, bc = x(Cc), torch.randn(Cc, 4, device=dev, dtype=dt), torch.randn(Cc, device=dev, dtype=dt)
        st = torch.zeros(batch, 3, Cc, device=dev, dtype=dt)
        ms = _time(lambda: M.short_conv_silu(xc, wc, st, meta, bias=bc), flush, graph=replay)
        rec("short_conv_silu(bias)", phase, ms, 2 * T * Cc * 2, 0, like="short_conv_silu")
        ms = _time(lambda: M.short_conv_silu(xc, wc, st, meta), flush, graph=replay)
        rec("gopunex:short_conv_silu", phase, ms, 2 * T * Cc * 2, 0)
        # gate-first group norm (state space), head norm (matrix memory)  |  like: the gated group norm
        o, gate, wn = torch.randn(T, 2 * width, device=dev), x(2 * width), torch.ones(2 * width, device=dev, dtype=dt)
        ms = _time(lambda: M.gated_group_rms_norm(o, wn, gate, 2 * width, 1e-6, dt, gate_act="silu", gate_first=True), flush,
                   graph=replay)
        rec("gated_group_rmsnorm(gate first, one group)", phase, ms, T * 2 * width * (4 + 2 + 2), 0, like="gated_group_rmsnorm")
        wh = torch.ones(d, device=dev, dtype=dt)
        ms = _time(lambda: M.gated_group_rms_norm(o, wh, gate, d, 1e-6, dt), flush, graph=replay)
        rec("gopunex:gated_group_rmsnorm", phase, ms, T * 2 * width * (4 + 2 + 2), 0)
        # rotary pairs + unit norm of q | k heads in place  |  like: Llama's in-place rotation
        L = ctx + q_len
        qkv = x((H + 2 * G) * d)
        tab = M.rotary_table(L, 64, 5e5, dev)
        ms = _time(lambda: M.rotary_unit_norm(qkv, H + G, d, 64, True, tab, meta.token_pos, 1e-6), flush, graph=replay)
        rec("rotary_unit_norm", phase, ms, 2 * T * (H + G) * d * 2, 0, like="rope_qkv")
        cos, sin = ops.build_rope_cache(L, d, 5e5, device=dev)
        posl = meta.token_pos.long()
        ms = _time(lambda: ops.rope_qkv(qkv, posl, cos, sin, H, G, d), flush, graph=replay)
        rec("llama:rope_qkv", phase, ms, 2 * T * (H + G) * d * 2, 0)
        og, gg = x(H * d), x(H * d)
        ms = _time(lambda: M.sigmoid_gate_mul(og, gg), flush, graph=replay)
        rec("sigmoid_gate_mul", phase, ms, 3 * T * H * d * 2, 0, like="glu_fwd(silu)")
        gu = x(2 * H * d)
        ms = _time(lambda: ops.glu(gu, "silu"), flush, graph=replay)
        rec("llama:glu_fwd(silu)", phase, ms, 3 * T * H * d * 2, 0)
        # attention over pages: causal and block-masked, both with two-term weights  |  like: bias + sink attention
        per = (L + bs - 1) // bs
        kc = torch.randn(batch * per, bs, G, d, device=dev, dtype=dt)
        vc = torch.randn(batch * per, bs, G, d, device=dev, dtype=dt)
        tables = torch.arange(batch * per, dtype=torch.int32, device=dev).view(batch, per)
        qa = x(H * d)
        kv_bytes = 2 * batch * L * G * d * 2
        att_flops = 4.0 * batch * H * d * (q_len * ctx + q_len * (q_len + 1) / 2)
        ms = _time(lambda: M.paged_bias_attention(qa, kc, vc, tables, meta, d ** -0.5, wide_weights=True), flush, graph=replay)
        # (rooflines count the algorithm's FLOPs: the second term of the weights is overhead, not work)
        rec("paged_attention(causal, two-term weights)", phase, ms, kv_bytes + 2 * T * H * d * 2, att_flops,
            like="paged_bias_attention")
        mb = 1024
        seen = sum(min(p_ % mb + 1, p_ + 1) for p_ in range(ctx, L)) * batch        # keys every query sees
        ms = _time(lambda: M.paged_bias_attention(qa, kc, vc, tables, meta, d ** -0.5, mask_block=mb, wide_weights=True),
                   flush, graph=replay)
        rec("paged_attention(blocks of 1024, two-term weights)", phase, ms,
            2 * batch * min(L, mb + q_len) * G * d * 2 + 2 * T * H * d * 2, 4.0 * H * d * seen,
            like="paged_bias_attention")
        rel = torch.randn(32, H, device=dev)
        starts_host = M.log_bucket_starts(32, 512.0)
        starts = torch.tensor(starts_host, dtype=torch.int32, device=dev)
        lut = M.bucket_lut(starts_host).to(dev)
        ms = _time(lambda: M.paged_bias_attention(qa, kc, vc, tables, meta, d ** -0.5, rel, starts, True, lut=lut), flush,
                   graph=replay)
        rec("gopunex:paged_bias_attention", phase, ms, kv_bytes + 2 * T * H * d * 2, att_flops)
    return rows


def kernels_domorax(width: int, batch: int, in_len: int, kv_rank: int = 192, rot: int = 64) -> list:
    """Every kernel of the Domorax layers alone at one layer's sizes beside its like kernel of the closest families."""
    from colossalai_b200 import ops
    from colossalai_b200.ops import mixers as M
    from colossalai_b200.ops import moe as MO

    hbm, tflops, src = peaks()
    dev, dt = "cuda", torch.bfloat16
    H, d, bs = width // 128, 128, 64
    G = max(H // 4, 1)
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    rows = []

    def rec(name, phase, ms, bytes_, flops, like=""):
        ideal = max(bytes_ / hbm, flops / tflops) * 1e3
        rows.append({"kernel": name, "phase": phase + ("(graph replay)" if phase == "decode" else ""), "width": width,
                     "ms": ms, "roofline_ms": ideal, "frac_of_" + src + "_roofline": ideal / ms,
                     "bound": "hbm" if bytes_ / hbm > flops / tflops else "tensor", "like": like})

    for phase, q_len, ctx in (("prefill", in_len, 0), ("decode", 1, in_len)):
        replay = phase == "decode"             # decode kernels are timed as graph replays (no host share)
        T = batch * q_len
        L = ctx + q_len
        meta = M.RaggedMeta.build([q_len] * batch, [ctx] * batch, list(range(batch)), dev)
        x = lambda c: torch.randn(T, c, device=dev, dtype=dt)
        # output norm in groups + scaled add, alone and with the depth average over 5 slices  |  like: Gopunex norm + residual
        n = 5
        hist = torch.randn(n + 1, T, width, device=dev)
        coef = torch.full((n,), 1.0 / n, device=dev)
        y1, w = x(width), torch.ones(width, device=dev, dtype=dt)
        ms = _time(lambda: M.rms_norm_residual(hist[n - 1], y1, w, 1e-5, 0.5, groups=4), flush, graph=replay)
        rec("rmsnorm_residual(4 groups)", phase, ms, T * width * (4 + 4 + 2 + 2), 0, like="rmsnorm_residual")
        ms = _time(lambda: M.rms_norm_residual(hist[n - 1], y1, w, 1e-5, 0.5, groups=4, history=(hist, n, coef, hist[n])),
                   flush, graph=replay)
        rec("rmsnorm_residual(4 groups) + depth average(5)", phase, ms, T * width * (2 + 4 + 4 + (n - 1) * 4 + 4 + 2), 0,
            like="rmsnorm_residual")
        yf = torch.randn(T, width, device=dev)
        ms = _time(lambda: M.rms_norm_residual(hist[n - 1], yf, w, 1e-5, 0.5, groups=4), flush, graph=replay)
        rec("rmsnorm_residual(4 groups, fp32 sum in)", phase, ms, T * width * (4 + 4 + 4 + 2), 0, like="rmsnorm_residual")
        xs = torch.randn(T, width, device=dev)
        ms = _time(lambda: M.rms_norm_residual(xs, y1, w, 1e-5, 0.7, 1.0), flush, graph=replay)
        rec("gopunex:rmsnorm_residual", phase, ms, T * width * (4 + 4 + 2 + 2), 0)
        # normalised powers  |  like: Llama's gated unit, the other elementwise pass over the feed-forward's hidden vector
        z, pc = x(4 * width), torch.tensor([0.6, 0.3, 0.1, 0.0], device=dev)
        ms = _time(lambda: M.poly_norm(z, pc, 1e-5), flush, graph=replay)
        rec("poly_norm", phase, ms, 2 * T * 4 * width * 2, 0, like="glu_fwd(silu)")
        gu = x(2 * 4 * width)
        ms = _time(lambda: ops.glu(gu, "silu"), flush, graph=replay)
        rec("llama:glu_fwd(silu)", phase, ms, 3 * T * 4 * width * 2, 0)
        # delta rule with one decay per head  |  like: Gopunex delta rule with a decay per channel
        Gd = max(H // 2, 1)
        S = torch.zeros(batch, H, d, d, device=dev)
        state_bytes = 2 * S.numel() * 4
        q, k, v, a1, b1 = x(Gd * d) * 0.1, x(Gd * d) * 0.1, x(H * d), x(H), x(H)
        al, db = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
        ms = _time(lambda: M.state_scan_delta(q, k, v, a1, b1, al, db, S, meta, H, Gd, d, d, head_decay=True), flush,
                   graph=replay)
        rec("state_scan_delta(decay per head)", phase, ms, T * ((2 * Gd + H) * d * 2 + H * d * 4) + state_bytes,
            6.0 * T * H * d * d, like="state_scan_delta")
        qg, kg, ag, dbg = x(H * d) * 0.1, x(H * d) * 0.1, x(H * d), torch.zeros(H * d, device=dev)
        ms = _time(lambda: M.state_scan_delta(qg, kg, v, ag, b1, al, dbg, S, meta, H, H, d, d), flush, graph=replay)
        rec("gopunex:state_scan_delta", phase, ms, T * (4 * H * d * 2 + H * d * 4) + state_bytes, 6.0 * T * H * d * d)
        # convolution on q | k without activation, per-head norm  |  like: Gopunex convolution, Llama's in-place rotation
        Cc = (H + G) * d
        xc, wc = x(Cc), torch.randn(Cc, 4, device=dev, dtype=dt)
        stc = torch.zeros(batch, 3, Cc, device=dev, dtype=dt)
        ms = _time(lambda: M.short_conv_silu(xc, wc, stc, meta, activation=False), flush, graph=replay)
        rec("short_conv(q | k, no activation)", phase, ms, 2 * T * Cc * 2, 0, like="short_conv_silu")
        ms = _time(lambda: M.short_conv_silu(xc, wc, stc, meta), flush, graph=replay)
        rec("gopunex:short_conv_silu", phase, ms, 2 * T * Cc * 2, 0)
        wh = torch.ones(d, device=dev, dtype=dt)
        ms = _time(lambda: M.head_rms_norm(xc, H, G, d, wh, wh, 1e-5), flush, graph=replay)
        rec("head_rms_norm(q | k)", phase, ms, 2 * T * Cc * 2, 0, like="rope_qkv")
        qkv = x((H + 2 * G) * d)
        cos, sin = ops.build_rope_cache(L + 1, d, 5e5, device=dev)
        pos = meta.token_pos.long()
        ms = _time(lambda: ops.rope_qkv(qkv, pos, cos, sin, H, G, d), flush, graph=replay)
        rec("llama:rope_qkv", phase, ms, 2 * T * (H + G) * d * 2, 0)
        o, gate, wn = torch.randn(T, H * d, device=dev), x(H * d), torch.ones(d, device=dev, dtype=dt)
        ms = _time(lambda: M.gated_group_rms_norm(o, wn, gate, d, 1e-5, dt, gate_act="silu"), flush, graph=replay)
        rec("gated_group_rmsnorm(silu)", phase, ms, T * H * d * (4 + 2 + 2), 0, like="gated_group_rmsnorm")
        # query latent norm, cache row of latent attention  |  like: Gopunex K / V page write
        qr = width * 3 // 8
        zq, wq = x(qr + kv_rank + rot), torch.ones(qr, device=dev, dtype=dt)
        ms = _time(lambda: M.head_rms_norm(zq, 1, 0, qr, wq, None, 1e-5), flush, graph=replay)
        rec("head_rms_norm(query latent)", phase, ms, 2 * T * qr * 2, 0, like="rmsnorm_fwd")
        per = (L + bs - 1) // bs
        W2 = kv_rank + rot
        lc = torch.randn(batch * per, bs, 1, W2, device=dev, dtype=dt)
        tables = torch.arange(batch * per, dtype=torch.int32, device=dev).view(batch, per)
        table = M.rotary_table(L + 1, rot, 5e5, dev, [4.0, 4096.0, 32.0, 1.0])
        wl = torch.ones(kv_rank, device=dev, dtype=dt)
        ms = _time(lambda: M.latent_kv_write(zq[:, qr:], wl, 1e-5, kv_rank, table, lc, tables, meta), flush, graph=replay)
        rec("latent_kv_write(stretched frequencies)", phase, ms, 2 * T * W2 * 2, 0, like="paged_kv_write_mix")
        # attention: latent rows with a window of 1024 and learned sinks; convolved attention with distance slopes (values
        # in a cache of their own); both with two-term weights  |  like: Palilix latent attention, Gopunex bias + sink
        win = 1024
        qa2 = x(H * W2)
        sinks = torch.randn(H, device=dev)
        seen = sum(min(p_ + 1, win) for p_ in range(ctx, L)) * batch                  # keys every query sees
        ms = _time(lambda: M.paged_bias_attention(qa2, lc, lc, tables, meta, d ** -0.5, vdim=kv_rank, window=win, sink=True,
                                                  sink_values=sinks, wide_weights=True), flush, graph=replay)
        rec("latent_attention(window 1024, sinks, two-term weights)", phase, ms,
            batch * min(L, win + q_len) * W2 * 2 + T * H * (W2 + kv_rank) * 2, 2.0 * H * (W2 + kv_rank) * seen,
            like="latent_attention")
        full = batch * (q_len * ctx + q_len * (q_len + 1) / 2)
        ms = _time(lambda: M.paged_bias_attention(qa2, lc, lc, tables, meta, d ** -0.5, vdim=kv_rank), flush, graph=replay)
        rec("palilix:latent_attention", phase, ms, batch * L * W2 * 2 + T * H * (W2 + kv_rank) * 2,
            2.0 * H * (W2 + kv_rank) * full)
        kc = torch.randn(batch * per, bs, G, d, device=dev, dtype=dt)
        vc = torch.randn(batch * per, bs, G, d, device=dev, dtype=dt)
        qa = x(H * d)
        slopes = M.distance_slopes(H).to(dev)
        kv_bytes = 2 * batch * L * G * d * 2
        att_flops = 4.0 * H * d * full
        ms = _time(lambda: M.paged_bias_attention(qa, kc, vc, tables, meta, d ** -0.5, slopes=slopes, wide_weights=True),
                   flush, graph=replay)
        rec("paged_attention(distance slopes, two-term weights)", phase, ms, kv_bytes + 2 * T * H * d * 2, att_flops,
            like="paged_bias_attention")
        rel = torch.randn(32, H, device=dev)
        starts_host = M.log_bucket_starts(32, 512.0)
        starts = torch.tensor(starts_host, dtype=torch.int32, device=dev)
        lut = M.bucket_lut(starts_host).to(dev)
        ms = _time(lambda: M.paged_bias_attention(qa, kc, vc, tables, meta, d ** -0.5, rel, starts, True, lut=lut), flush,
                   graph=replay)
        rec("gopunex:paged_bias_attention", phase, ms, kv_bytes + 2 * T * H * d * 2, att_flops)
        # fp32 gather of the chosen experts' rows + the gated shared expert  |  like: Palilix gather
        ys, sh = x(width).repeat(2, 1), x(width)
        row_of = torch.randperm(2 * T, device=dev).view(T, 2)
        wts, sg = torch.rand(T, 2, device=dev), torch.randn(T, 9, device=dev)[:, 8]
        ms = _time(lambda: MO.gather_combine(ys, row_of, wts, extra=sh, extra_gate=sg), flush, graph=replay)
        rec("moe_gather_combine(+ gated shared expert)", phase, ms, T * width * (3 * 2 + 4), 0, like="moe_gather_combine")
        ms = _time(lambda: MO.gather_combine(ys, row_of, wts), flush, graph=replay)
        rec("palilix:moe_gather_combine", phase, ms, T * width * (2 * 2 + 4), 0)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="2048x8,4096x4", help="width x layers, comma separated")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--in_len", type=int, default=2048)
    ap.add_argument("--out_len", type=int, default=32)
    ap.add_argument("--cuda_graph", action="store_true", help="also run both families with CUDA-graph decode steps")
    ap.add_argument("--family", default="gopunex", choices=["gopunex", "palilix", "pogorax", "domorax"],
                    help="gopunex: the hybrid decoder beside Llama (default).  palilix / pogorax / domorax: that family "
                         "beside Gopunex, the closest served family")
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--no-serve", action="store_true")
    args = ap.parse_args(argv)
    assert torch.cuda.is_available(), "this benchmark needs a GPU"
    for size in args.sizes.split(","):
        width, layers = (int(z) for z in size.split("x"))
        if not args.no_serve:
            for graph in ([False, True] if args.cuda_graph else [False]):
                pair = {"gopunex": lambda: (hybrid_config(width, layers), llama_config(width, layers)),
                        "palilix": lambda: (palilix_config(width, layers), hybrid_config(width, layers)),
                        "pogorax": lambda: (pogorax_config(width, layers), hybrid_config(width, layers)),
                        "domorax": lambda: (domorax_config(width, layers), hybrid_config(width, layers))}[args.family]()
                for cfg in pair:
                    print(json.dumps(serve(cfg, args.batch, args.in_len, args.out_len, graph)), flush=True)
        if not args.no_kernels:
            kfn = {"gopunex": kernels, "palilix": kernels_palilix, "pogorax": kernels_pogorax,
                   "domorax": kernels_domorax}[args.family]
            for row in kfn(width, args.batch, args.in_len):
                print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
