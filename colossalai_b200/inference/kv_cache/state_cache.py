"""Fixed-size recurrent state per live sequence, beside the paged K / V of attention layers.

A recurrent mixer (linear attention, retention, delta rule, selective state space, gated matrix memory, gated linear
recurrence; also attention whose q / k pass a short convolution, which carries the convolution's window only) keeps, per sequence, fp32 memories ("S" and, for the gated matrix memory, the normaliser "n" and the running
maximum "m") and - where it has short convolutions - the last few inputs of every convolved channel ("conv", in the
compute dtype).  A layer whose mixer is a pair of mixers holds the pages of its paged part and the state of its recurrent
part.  The pool holds `max_batch_size` slots per such
layer; a sequence takes a slot when it is admitted and gives it back when it ends.  Slots are not cleared: the kernels
take the state of a sequence that has consumed no token yet as zero.

Caches and states are indexed by LAYER RUN (`cache_layers`): a layer inside a looped span runs several times per forward
with the same weights, and every pass owns pages / slots of its own.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ...accelerator import get_accelerator

__all__ = ["StateCacheManager", "layer_cache_shapes", "layer_state_shapes", "cache_layers"]


def cache_layers(model_config) -> List[int]:
    """Layer index of every layer run, in execution order (one cache / state per run)."""
    runs = getattr(model_config, "layer_runs", None)
    if runs is None:
        return list(range(model_config.num_hidden_layers))
    return [layer for layer, _ in runs()]


def _spec(model_config, layer: int):
    specs = getattr(model_config, "layer_specs", None)
    return None if specs is None else specs[layer].mixer


def layer_cache_shapes(model_config, layer: int, num_blocks: int, block_size: int,
                       tp_size: int = 1) -> Optional[Tuple[Tuple[int, ...], Optional[Tuple[int, ...]]]]:
    """(K shape, V shape) of a layer's paged cache, None for a layer without one.  Latent attention keeps ONE row per
    token, [latent | rotated key part]; its values are the latent columns of the same row (V shape None)."""
    sp = _spec(model_config, layer)
    if sp is None:
        kv = max(getattr(model_config, "num_key_value_heads", model_config.num_attention_heads) // tp_size, 1)
        shp = (num_blocks, block_size, kv, model_config.head_dim)
        return shp, shp
    sp = sp.paged_part
    if sp is None:
        return None
    if sp.kind == "latent":
        return (num_blocks, block_size, 1, sp.kv_rank + sp.rot_dim), None
    if sp.kind != "attention":
        return None
    return (num_blocks, block_size, sp.kv_heads, sp.dim), (num_blocks, block_size, sp.kv_heads, sp.vdim)


def layer_state_shapes(model_config, layer: int, slots: int) -> Optional[Dict[str, Tuple[int, ...]]]:
    """Shapes of a recurrent layer's state tensors ("S", "n", "m": fp32 memories; "conv": carried convolution inputs in
    the compute dtype)."""
    sp = _spec(model_config, layer)
    sp = None if sp is None else sp.recurrent_part
    if sp is None:
        return None
    if sp.kind == "attention":            # attention behind a convolution on q | k: only the convolution's window
        return {"conv": (slots, max(sp.conv - 1, 0), (sp.heads + sp.kv_heads) * sp.dim)}
    if sp.kind == "rglru":
        return {"S": (slots, sp.lru_width), "conv": (slots, max(sp.conv - 1, 0), sp.lru_width)}
    if sp.kind == "ssd":
        return {"S": (slots, sp.heads, sp.state, sp.vdim),
                "conv": (slots, max(sp.conv - 1, 0), sp.heads * sp.vdim + 2 * sp.groups * sp.state)}
    out = {"S": (slots, sp.heads, sp.dim, sp.vdim)}
    if sp.kind == "mlstm":
        out["n"], out["m"] = (slots, sp.heads, sp.dim), (slots, sp.heads)
    if sp.kind in ("channel_delta", "delta"):        # a one-tap convolution carries nothing: an empty tensor keeps the call uniform
        out["conv"] = (slots, max(sp.conv - 1, 0), 2 * sp.kv_heads * sp.dim + sp.heads * sp.vdim)
    return out


class StateCacheManager:
    def __init__(self, config, model_config) -> None:
        self.device = get_accelerator().get_current_device()
        self.num_slots = config.max_batch_size
        self.dtype = config.dtype
        self._free: List[int] = list(range(self.num_slots))
        self.states: List[Optional[Dict[str, torch.Tensor]]] = []
        for i in cache_layers(model_config):                  # models without recurrent layers only use the slot ids
            shapes = layer_state_shapes(model_config, i, self.num_slots)
            self.states.append(None if shapes is None else {
                n: torch.zeros(s, dtype=self.dtype if n.startswith("conv") else torch.float32, device=self.device)
                for n, s in shapes.items()})

    @property
    def num_available_slots(self) -> int:
        return len(self._free)

    @property
    def has_state(self) -> bool:
        return any(s is not None for s in self.states)

    def allocate(self) -> int:
        if not self._free:
            raise RuntimeError("No state slot available.")
        return self._free.pop(0)

    def free(self, slot: int) -> None:
        assert 0 <= slot < self.num_slots and slot not in self._free
        self._free.append(slot)

    def total_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for s in self.states if s is not None for t in s.values())
