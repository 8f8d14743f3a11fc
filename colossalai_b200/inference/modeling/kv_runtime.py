"""Runtime object handed to the model as `kv_cache`: writes K/V into the paged cache and runs attention.

Replaces the reference's no-padding model forwards + attention backends (`inference/modeling/models/nopadding_llama.py`,
`modeling/backends/{attention_backend,pre_attention_backend}.py`): our generic model already works on flattened
un-padded tokens, so inference only has to (a) scatter the step's K/V into the block tables and (b) run varlen
flash-attention for prefill or the paged split-KV kernel for decode.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ... import ops
from ...ops import inference as iops

__all__ = ["PagedKVRuntime"]


class PagedKVRuntime:
    def __init__(self, k_caches: List[torch.Tensor], v_caches: List[torch.Tensor], block_size: int,
                 states: Optional[List[Optional[dict]]] = None) -> None:
        self.k_caches, self.v_caches = k_caches, v_caches
        self.block_size = block_size
        self.states = states                                  # per layer: recurrent state tensors indexed by slot
        self.ragged = None                                    # ops.mixers.RaggedMeta of the step (ragged steps)
        self.shared: dict = {}                                # tensors one layer lends to later ones within a step
        self.run_of: dict = {}                                # layer -> cache index of its current run (looped spans)
        self.block_tables: Optional[torch.Tensor] = None      # [bsz, max_blocks] int32 (device)
        self.seq_lens: Optional[torch.Tensor] = None          # [bsz] int32, INCLUDING the tokens of this step
        self.is_prompt = True
        self.token_seq: Optional[torch.Tensor] = None         # [tokens] int32 sequence index of every token
        self.token_pos: Optional[torch.Tensor] = None         # [tokens] int32 position of every token
        self.cu_seqlens: Optional[torch.Tensor] = None
        self.max_seqlen: int = 0
        self.q_per_seq: int = 1                               # decode: tokens verified per sequence (spec-dec)
        self.max_len_host: int = 0                            # longest sequence of the step (host side, no sync)

    def set_step(self, block_tables: torch.Tensor, seq_lens: torch.Tensor, is_prompt: bool, device,
                 q_per_seq: int = 1) -> torch.Tensor:
        """Prepare per-step metadata; returns the int64 position of every input token."""
        self.block_tables = block_tables.to(device=device, dtype=torch.int32).contiguous()
        self.seq_lens = seq_lens.to(device=device, dtype=torch.int32).contiguous()
        self.ragged = None
        self.is_prompt = is_prompt
        self.q_per_seq = q_per_seq
        lens = seq_lens.tolist()
        self.max_len_host = max(lens) if lens else 0
        if is_prompt:
            seq = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens))
            pos = torch.cat([torch.arange(l) for l in lens])
            cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
            cu[1:] = torch.cumsum(torch.tensor(lens), 0)
            self.cu_seqlens = cu.to(device)
            self.max_seqlen = max(lens)
        else:
            seq = torch.repeat_interleave(torch.arange(len(lens)), q_per_seq)
            pos = torch.cat([torch.arange(l - q_per_seq, l) for l in lens])
            self.cu_seqlens = None
        self.token_seq = seq.to(device=device, dtype=torch.int32)
        self.token_pos = pos.to(device=device, dtype=torch.int32)
        return pos.to(device=device, dtype=torch.int64)

    # ------------------------------------------------------------------ ragged steps (portions + decoded tokens)
    def set_ragged_step(self, block_tables: torch.Tensor, q_lens, ctx_lens, slots, device) -> torch.Tensor:
        """A step in which sequence i brings `q_lens[i]` new tokens on top of `ctx_lens[i]` cached ones: whole prompts,
        portions of prompts and single decoded tokens side by side.  Returns the int64 position of every token."""
        from ...ops.mixers import RaggedMeta

        self.ragged = RaggedMeta.build(q_lens, ctx_lens, slots, device)
        self.block_tables = block_tables.to(device=device, dtype=torch.int32).contiguous()
        self.token_seq, self.token_pos = self.ragged.token_seq, self.ragged.token_pos
        self.seq_lens = self.ragged.ctx_len + (self.ragged.cu_q[1:] - self.ragged.cu_q[:-1])
        self.is_prompt, self.q_per_seq, self.cu_seqlens = False, 1, None
        self.max_len_host = max((c + n for c, n in zip(self.ragged.ctx_lens, self.ragged.q_lens)), default=0)
        self.shared = {}
        return self.token_pos.long()

    def set_ragged_static(self, flat: torch.Tensor, block_tables: torch.Tensor, nseq: int, max_ctx: int) -> torch.Tensor:
        """Decode step over fixed device buffers (what a CUDA graph of the step captures and replays)."""
        from ...ops.mixers import RaggedMeta

        self.ragged = RaggedMeta.decode_static(flat, nseq, max_ctx)
        self.block_tables = block_tables
        self.token_seq, self.token_pos = self.ragged.token_seq, self.ragged.token_pos
        self.seq_lens = self.ragged.ctx_len + 1
        self.is_prompt, self.q_per_seq, self.cu_seqlens = False, 1, None
        self.max_len_host = max_ctx + 1
        self.shared = {}
        return self.token_pos.long()

    def bind_run(self, layer_idx: int, run_idx: int) -> None:
        """The backbone names the layer run that is about to execute: a layer inside a looped span has one cache /
        state per pass, stored at the run's index."""
        self.run_of[layer_idx] = run_idx

    def cache_index(self, layer_idx: int) -> int:
        return self.run_of.get(layer_idx, layer_idx)

    def layer_state(self, layer_idx: int) -> dict:
        return self.states[self.cache_index(layer_idx)]

    def attend_latent(self, layer_idx: int, q: torch.Tensor, scale: float, kv_rank: int, window: int = 0,
                      sink: bool = False, sink_values: Optional[torch.Tensor] = None,
                      wide_weights: bool = False) -> torch.Tensor:
        """Latent attention over the layer's pages (rows [latent | rotated key part], written by the caller through
        `latent_cache`): q [T, H x (kv_rank + rot)] against the whole row, values = the row's first `kv_rank` columns;
        optionally inside a sliding `window` and with a sink (`sink_values`: its score per head) in the denominator.
        Returns [T, H x kv_rank]."""
        from ...ops import mixers as mops

        kc = self.k_caches[self.cache_index(layer_idx)]
        return mops.paged_bias_attention(q, kc, kc, self.block_tables, self.ragged, scale, vdim=kv_rank, window=window,
                                         sink=sink, sink_values=sink_values, wide_weights=wide_weights)

    def pages(self, layer_idx: int):
        """(key pages, value pages) of the layer's current run, for a mixer whose kernels write the step's rows themselves."""
        return self.k_caches[self.cache_index(layer_idx)], self.v_caches[self.cache_index(layer_idx)]

    def latent_cache(self, layer_idx: int) -> torch.Tensor:
        return self.k_caches[self.cache_index(layer_idx)]

    def attend_ragged(self, layer_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                      bias_table=None, bucket_starts=None, sink: bool = False, v_other=None,
                      lam: float = 0.0, lut=None, mask_block: int = 0, wide_weights: bool = False,
                      sink_values: Optional[torch.Tensor] = None, slopes: Optional[torch.Tensor] = None,
                      window: int = 0) -> torch.Tensor:
        """Write the step's K / V rows (values optionally blended with `v_other`) into the layer's pages, then attend
        every step token over positions 0..pos of its sequence (with `mask_block`: over the positions of its own block
        of that many positions only; with `window`: over the last `window` positions; `slopes`: a linear distance
        penalty per head; `sink_values`: the sink's score per head).  q [T, H x dim], k [T, G x dim], v [T, G x vdim];
        k = None: the caller has written the step's rows itself (`pages`)."""
        from ...ops import mixers as mops

        kc, vc = self.k_caches[self.cache_index(layer_idx)], self.v_caches[self.cache_index(layer_idx)]
        if k is not None:
            mops.paged_kv_write_mix(k, v, kc, vc, self.block_tables, self.ragged, v_other=v_other, lam=lam)
        return mops.paged_bias_attention(q, kc, vc, self.block_tables, self.ragged, scale, bias_table=bias_table,
                                         bucket_starts=bucket_starts, sink=sink, lut=lut, mask_block=mask_block,
                                         wide_weights=wide_weights, sink_values=sink_values, slopes=slopes, window=window)

    @classmethod
    def scratch(cls, cfg, batch: int, seqlen: int, device, dtype, block_size: int = 16) -> "PagedKVRuntime":
        """Cache pages and state slots for `batch` fresh sequences of `seqlen` tokens, laid out back to back: what a
        forward without a serving engine runs on."""
        from ..kv_cache.state_cache import cache_layers, layer_cache_shapes, layer_state_shapes

        per = (seqlen + block_size - 1) // block_size
        ks, vs, states = [], [], []
        for i in cache_layers(cfg):
            shp = layer_cache_shapes(cfg, i, batch * per, block_size)
            ks.append(None if shp is None else torch.zeros(shp[0], dtype=dtype, device=device))
            vs.append(None if shp is None or shp[1] is None else torch.zeros(shp[1], dtype=dtype, device=device))
            st = layer_state_shapes(cfg, i, batch)
            states.append(None if st is None else {
                n: torch.zeros(sh, dtype=dtype if n.startswith("conv") else torch.float32, device=device)
                for n, sh in st.items()})
        rt = cls(ks, vs, block_size, states)
        tables = torch.arange(batch * per, dtype=torch.int32).view(batch, per)
        rt.set_ragged_step(tables, [seqlen] * batch, [0] * batch, list(range(batch)), device)
        return rt

    def attend(self, layer_idx: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta, scale: float,
               alibi_slopes: Optional[torch.Tensor] = None, sliding_window: Optional[int] = None) -> torch.Tensor:
        if self.ragged is not None:
            # a ragged step (portions of prompts beside decoded tokens): rotary / plain attention families take the same
            # paged kernels as the hybrid decoders, without bias table and sink
            if alibi_slopes is not None or sliding_window is not None:
                raise NotImplementedError("ragged steps (chunked prefill) do not cover ALiBi or sliding-window attention")
            T, hq = q.shape[0], q.shape[1]
            o = self.attend_ragged(layer_idx, q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), scale)
            return o.view(T, hq, -1)
        kc, vc = self.k_caches[self.cache_index(layer_idx)], self.v_caches[self.cache_index(layer_idx)]
        iops.kv_cache_write(k, v, kc, vc, self.block_tables, self.token_seq, self.token_pos)
        if sliding_window is not None and self.max_len_host > sliding_window:
            return self._attend_windowed(q, k, v, kc, vc, scale, alibi_slopes, sliding_window)
        return self._attend_full(q, k, v, kc, vc, scale, alibi_slopes)

    def _native_prefill(self, q, k, v, scale, window: int, alibi_slopes) -> Optional[torch.Tensor]:
        """Sliding-window / ALiBi prefill inside the tcgen05 flash kernel (packed batch, device-resident boundaries);
        None when the tensors are outside the kernel's envelope (CPU tests, head_dim other than 64 / 128, fp32)."""
        from ...ops import flash_attn_native as fan

        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        if not fan.supported(q, k, v, self.cu_seqlens, self.cu_seqlens, force=True):
            return None
        return fan.flash_prefill(q, k, v, self.cu_seqlens, scale, window=window, alibi_slopes=alibi_slopes)

    def _attend_windowed(self, q, k, v, kc, vc, scale, alibi_slopes, window: int) -> torch.Tensor:
        """Sliding-window attention (Mistral): a sequence longer than the window takes the banded reference path —
        prefill with an explicit band mask per sequence, decode over the last `window` cached tokens."""
        from ...ops.attention import attention_ref

        if self.is_prompt:
            native = self._native_prefill(q, k, v, scale, window, alibi_slopes)
            if native is not None:
                return native
            cu = self.cu_seqlens.tolist()
            outs = []
            for i in range(len(cu) - 1):
                a, b = cu[i], cu[i + 1]
                S = b - a
                pos = torch.arange(S, device=q.device)
                rel = pos[None, :] - pos[:, None]
                keep = (rel <= 0) & (rel > -window)
                bias = torch.zeros(S, S, device=q.device, dtype=torch.float32)
                if alibi_slopes is not None:
                    bias = rel.clamp(max=0).float()[None] * alibi_slopes.float()[:, None, None]
                bias = bias.expand(q.shape[1], S, S) if bias.dim() == 3 else bias[None].expand(q.shape[1], S, S)
                bias = bias.masked_fill(~keep[None], float("-inf")).to(q.dtype)[None]
                outs.append(attention_ref(q[a:b], k[a:b], v[a:b], batch=1, causal=False, scale=scale, attn_mask=bias))
            return torch.cat(outs, 0)
        n = self.q_per_seq
        if n == 1:
            return iops.paged_decode_attention(q, kc, vc, self.block_tables, self.seq_lens, scale,
                                               alibi_slopes=alibi_slopes, window=window)
        bsz = self.seq_lens.numel()
        outs = []
        for j in range(n):
            qj = q.view(bsz, n, *q.shape[1:])[:, j]
            outs.append(iops.paged_decode_attention(qj.contiguous(), kc, vc, self.block_tables,
                                                    self.seq_lens - (n - 1 - j), scale, alibi_slopes=alibi_slopes,
                                                    window=window))
        return torch.stack(outs, 1).reshape(q.shape)

    def _attend_full(self, q, k, v, kc, vc, scale, alibi_slopes) -> torch.Tensor:
        if alibi_slopes is not None:
            # ALiBi families (Baichuan-13B, BLOOM): biased varlen prefill through the reference backend, the paged
            # decode kernel takes the slopes natively
            from .backends.attention_backend import AttentionMetaData, ReferenceAttentionBackend

            if self.is_prompt:
                native = self._native_prefill(q, k, v, scale, 0, alibi_slopes)
                if native is not None:
                    return native
                md = AttentionMetaData(q, k, v, kc, vc, self.block_tables, self.block_size, cu_seqlens=self.cu_seqlens,
                                       sm_scale=scale, alibi_slopes=alibi_slopes)
                return ReferenceAttentionBackend().prefill(md)
            assert self.q_per_seq == 1, "speculative verification is not implemented for ALiBi models"
            return iops.paged_decode_attention(q, kc, vc, self.block_tables, self.seq_lens, scale,
                                               alibi_slopes=alibi_slopes)
        if self.is_prompt:
            return ops.attention(q, k, v, causal=True, scale=scale, cu_seqlens_q=self.cu_seqlens,
                                 cu_seqlens_k=self.cu_seqlens, max_seqlen=self.max_seqlen)
        if self.q_per_seq == 1:
            return iops.paged_decode_attention(q, kc, vc, self.block_tables, self.seq_lens, scale)
        # speculative verification: n query tokens per sequence, each sees the cache up to its own position
        n = self.q_per_seq
        bsz = self.seq_lens.numel()
        outs = []
        for j in range(n):
            qj = q.view(bsz, n, *q.shape[1:])[:, j]
            outs.append(iops.paged_decode_attention(qj.contiguous(), kc, vc, self.block_tables,
                                                    self.seq_lens - (n - 1 - j), scale))
        return torch.stack(outs, 1).reshape(q.shape)
