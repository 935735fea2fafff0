"""A model: embedding, a set of blocks, the order in which they run, and the output head.

The order is data. `schedule` is a list of `LayerCall(block, cache_layer, writes)`:
a block may appear more than once (weight sharing), and a call may read the cache
layer that another call fills (`writes=False`). Cache layers are numbered per model;
the cache manager groups those with equal needs. A mixer made of several mixers has a cache layer per
member (`cache_layer` a tuple, the block's `cache_spec()` a tuple of as many specs), and an embedding that
keeps something per request (`cache_spec()` not None) gets a cache layer after the blocks'.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..parts.base import Part


@dataclass(frozen=True)
class LayerCall:
    block: int          # index into Model.blocks
    cache_layer: int | tuple    # which cache layer the mixer uses (-1: none); a tuple: one per member of the mixer
    writes: bool = True  # False: read what another call wrote, write nothing

    @property
    def cache_layers(self) -> tuple:
        """The call's cache layers as a tuple (empty: none)."""
        if isinstance(self.cache_layer, tuple):
            return self.cache_layer
        return () if self.cache_layer < 0 else (self.cache_layer,)


class Model:
    def __init__(self, config, embedding: Part, blocks: list[Part], schedule: list[LayerCall],
                 head: Part, prefix: str = "model."):
        self.config = config
        self.embedding, self.blocks, self.schedule, self.head = embedding, blocks, schedule, head
        self.prefix = prefix
        for call in schedule:
            if not 0 <= call.block < len(blocks):
                raise ValueError(f"schedule names block {call.block}, model has {len(blocks)}")
        self.num_cache_layers = 1 + max((l for c in schedule for l in c.cache_layers), default=-1)
        writers = {l for c in schedule if c.writes for l in c.cache_layers}
        for c in schedule:
            for l in c.cache_layers:
                if l not in writers:
                    raise ValueError(f"cache layer {l} is read but never written")
        # an embedding with per-request state of its own takes the cache layer after the blocks'
        self.embedding_cache_layer = -1
        if embedding.cache_spec() is not None:
            self.embedding_cache_layer = self.num_cache_layers
            self.num_cache_layers += 1

    # -- structure
    def parts(self):
        yield from self.embedding.walk()
        for b in self.blocks:
            yield from b.walk()
        yield from self.head.walk()

    def cache_specs(self):
        """cache layer -> spec, from the block that writes it."""
        specs = {}
        for c in self.schedule:
            if not c.cache_layers or not c.writes:
                continue
            spec = self.blocks[c.block].cache_spec()
            members = spec if isinstance(c.cache_layer, tuple) else (spec,)
            if not isinstance(members, tuple) or len(members) != len(c.cache_layers):
                raise ValueError(f"block {c.block} needs {len(members) if isinstance(members, tuple) else 1} cache "
                                 f"layer(s), its call names {len(c.cache_layers)}")
            for l, sp in zip(c.cache_layers, members):
                if l in specs and specs[l] != sp:
                    raise ValueError(f"cache layer {l} is written with two different specs")
                specs[l] = sp
        if self.embedding_cache_layer >= 0:
            specs[self.embedding_cache_layer] = self.embedding.cache_spec()
        return [specs[i] for i in range(self.num_cache_layers)]

    @property
    def vocab_size(self) -> int:
        return self.head.vocab

    def finalize(self, device, dtype):
        for p in self.parts():
            p.finalize(device, dtype)

    # -- running
    def forward(self, ctx, caches):
        """Run the step's tokens through every scheduled layer -> float32 [T, hidden]."""
        if hasattr(ctx, "per_forward"):
            ctx.per_forward.clear()
        if self.embedding_cache_layer >= 0:
            h = self.embedding.forward(ctx, caches.layer_view(self.embedding_cache_layer, ctx, True))
        else:
            h = self.embedding.forward(ctx)
        for call in self.schedule:
            if isinstance(call.cache_layer, tuple):
                cache = tuple(caches.layer_view(l, ctx, call.writes) for l in call.cache_layer)
            else:
                cache = caches.layer_view(call.cache_layer, ctx, call.writes) if call.cache_layer >= 0 else None
            self.blocks[call.block].forward(h, ctx, cache)
        return h

    def logits(self, h, rows, ctx):
        return self.head.forward(h, rows, ctx)
