"""Device tensors behind the cache groups (see layout.py for the layout)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .layout import CacheLayout, KVLayerSpec, LatentLayerSpec, StateLayerSpec, flatten_specs


@dataclass
class CacheLayerView:
    """What a mixer sees of its cache layer during one step."""

    group: int  # index into CacheLayout.groups
    paged_index: int | None  # index among paged groups (selects the block table)
    page_size: int
    window: int | None
    k_pages: torch.Tensor | None  # [pages + 1, kv_heads, page_size, head_dim]
    v_pages: torch.Tensor | None
    state: torch.Tensor | None  # [slots + 1, *shape]
    writes: bool = True
    latent_pages: torch.Tensor | None = None  # [pages + 1, page_size, width] (a latent group)


class CacheStorage:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages: int | list[int], num_slots: int,
                 dtype: torch.dtype, device: torch.device | str):
        """``num_pages``: pages of every paged group, or one count per paged group."""
        self.layout = layout
        self.page_size = page_size
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(layout.paged_groups)
        if len(num_pages) != len(layout.paged_groups):
            raise ValueError("one page count per paged group is required")
        self.num_pages = list(num_pages)
        self.num_slots = num_slots
        # the extra page of each paged group, which padded rows write to
        self.scratch_page = tuple(self.num_pages)
        self.scratch_slot = num_slots
        self.tensors: list[torch.Tensor] = []
        for gi, g in enumerate(layout.groups):
            s = g.layer_spec
            if isinstance(s, KVLayerSpec) and s.split:  # keys and values of unlike sizes: a tensor each
                pages = self.num_pages[layout.paged_groups.index(gi)]
                shape = (len(g.cache_ids), pages + 1, s.num_kv_heads, page_size)
                self.tensors.append((torch.zeros((*shape, s.head_dim), dtype=dtype, device=device),
                                     torch.zeros((*shape, s.value_dim), dtype=dtype, device=device)))
            elif isinstance(s, KVLayerSpec):
                pages = self.num_pages[layout.paged_groups.index(gi)]
                shape = (len(g.cache_ids), 2, pages + 1, s.num_kv_heads, page_size, s.head_dim)
                self.tensors.append(torch.zeros(shape, dtype=dtype, device=device))
            elif isinstance(s, LatentLayerSpec):
                pages = self.num_pages[layout.paged_groups.index(gi)]
                shape = (len(g.cache_ids), pages + 1, page_size, s.width)
                self.tensors.append(torch.zeros(shape, dtype=dtype, device=device))
            else:
                assert isinstance(s, StateLayerSpec)
                shape = (len(g.cache_ids), num_slots + 1, *s.shape)
                self.tensors.append(torch.zeros(shape, dtype=getattr(torch, s.dtype), device=device))

    def view(self, cache_id, writes: bool = True):
        """What the mixer of one run entry sees: a :class:`CacheLayerView`, None (no cache), or, for a
        mixer whose spec is a tuple of specs, views in the same (possibly nested) arrangement."""
        if cache_id in self.layout.composite:
            leaves = iter(range(len(flatten_specs(self.layout.composite[cache_id]))))

            def arrange(spec):
                if isinstance(spec, (tuple, list)):
                    return tuple(arrange(part) for part in spec)
                return self.view((cache_id, next(leaves)), writes)

            return arrange(self.layout.composite[cache_id])
        if cache_id not in self.layout.where:
            return None
        gi, li = self.layout.where[cache_id]
        g = self.layout.groups[gi]
        t = self.tensors[gi]
        if isinstance(t, tuple):
            return CacheLayerView(gi, self.layout.paged_groups.index(gi), self.page_size, g.spec.window,
                                  t[0][li], t[1][li], None, writes)
        if g.spec.paged and isinstance(g.layer_spec, LatentLayerSpec):
            return CacheLayerView(gi, self.layout.paged_groups.index(gi), self.page_size, g.spec.window,
                                  None, None, None, writes, latent_pages=t[li])
        if g.spec.paged:
            return CacheLayerView(gi, self.layout.paged_groups.index(gi), self.page_size, g.spec.window,
                                  t[li, 0], t[li, 1], None, writes)
        return CacheLayerView(gi, None, self.page_size, None, None, None, t[li], writes)

    def zero_state_slots(self, slots: list[int]) -> None:
        """Fixed-size state starts from zero when a request starts or restarts."""
        if not slots:
            return
        idx = None
        for g, t in zip(self.layout.groups, self.tensors):
            if g.spec.paged:
                continue
            if idx is None:
                idx = torch.tensor(slots, dtype=torch.long, device=t.device)
            t.index_fill_(1, idx, 0)

    def poison_pages(self, paged_index: int, pages: list[int], value: float = float("nan")) -> None:
        """Overwrite pages (tests: a page that is used again must not leak old contents)."""
        gi = self.layout.paged_groups[paged_index]
        t = self.tensors[gi]
        if pages and isinstance(t, tuple):
            for part in t:
                part[:, torch.tensor(pages, dtype=torch.long, device=part.device)] = value
        elif pages and isinstance(self.layout.groups[gi].layer_spec, LatentLayerSpec):
            t[:, torch.tensor(pages, dtype=torch.long, device=t.device)] = value
        elif pages:
            t[:, :, torch.tensor(pages, dtype=torch.long, device=t.device)] = value

    def nbytes(self) -> int:
        flat = [x for t in self.tensors for x in (t if isinstance(t, tuple) else (t,))]
        return sum(t.numel() * t.element_size() for t in flat)
