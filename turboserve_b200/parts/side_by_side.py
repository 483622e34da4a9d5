"""Two mixers side by side on the same input, their outputs normed and added.

``out = weight_left * norm_left(left(h)) + weight_right * norm_right(right(h))``: each mixer's output is divided by
its root mean square over the model width (``eps`` inside the root) and multiplied by a weight of its own
(``left_norm`` and ``right_norm``, plain weights), in one kernel in fp32. The two mixers are parts of any registered
kind, given as ``left`` and ``right`` (``{"kind", "params"}``); their tensors carry the prefixes ``left_prefix`` and
``right_prefix``. What they keep per request is kept together: at most one of them may keep pages, and their
fixed-size states follow one another in the run's state list, the left mixer's first.
"""

from __future__ import annotations

from types import SimpleNamespace

import torch

from ..config.model_spec import PartSpec
from ..ops import kernels
from .base import MIXERS, Mixer, ParamSpec, register_mixer


def _part_spec(value) -> PartSpec:
    return value if isinstance(value, PartSpec) else PartSpec(value["kind"], dict(value.get("params") or {}))


class SideBySide(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device: torch.device | str,
                 position: PartSpec | None = None, shares_cache: bool = False) -> None:
        if shares_cache:
            raise ValueError("two mixers side by side keep caches of their own")
        self.hidden_size = int(hidden_size)
        self.eps = float(spec["eps"])
        self.weights = (float(spec.get("weight_left", 0.5)), float(spec.get("weight_right", 0.5)))
        self.prefixes = (str(spec.get("left_prefix", "left.")), str(spec.get("right_prefix", "right.")))
        self.norm_names = (str(spec.get("left_norm", "left.out")), str(spec.get("right_norm", "right.out")))
        self.sides: list[Mixer] = []
        for key in ("left", "right"):
            part = _part_spec(spec[key])
            self.sides.append(MIXERS.get(part.kind)(part, hidden_size, dtype, device, position=None, shares_cache=False))
        self.graph_safe = all(side.graph_safe for side in self.sides)
        from ..cache.storage import split_needs  # (that module reads this package's base on import)

        needs = [split_needs(side.cache_need()) for side in self.sides]
        if sum(1 for pages, _ in needs if pages is not None) > 1:
            raise ValueError("only one of two mixers side by side may keep pages")
        self._needs = needs
        self.gains: list[torch.Tensor | None] = [None, None]

    def cache_need(self):
        items = [pages for pages, _ in self._needs if pages is not None]
        for _, states in self._needs:
            items.extend(states)
        return tuple(items) if items else None

    def scratch_per_token(self) -> int | None:
        total = self.hidden_size
        for side in self.sides:
            own = side.scratch_per_token()
            if own is None:
                return None
            total += int(own)
        return total

    def param_specs(self) -> list[ParamSpec]:
        specs = []
        for side, prefix in zip(self.sides, self.prefixes):
            specs += [ParamSpec(prefix + p.name, p.shape, p.role, p.init) for p in side.param_specs()]
        specs += [ParamSpec(name, (self.hidden_size,), role="gain", init="one_plus_normal") for name in self.norm_names]
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for side, prefix in zip(self.sides, self.prefixes):
            side.bind({p.name: tensors[prefix + p.name] for p in side.param_specs()})
        self.gains = [tensors[name].contiguous() for name in self.norm_names]

    def _cache_of(self, index: int, cache):
        """The part of the run's cache that side ``index`` declared: the pages if it keeps some, and its own states."""
        first = sum(len(states) for _, states in self._needs[:index])
        pages, states = self._needs[index]
        return SimpleNamespace(
            kind="paged" if pages is not None else "state", group=cache.group, writes=cache.writes,
            k_pages=cache.k_pages if pages is not None else None, v_pages=cache.v_pages if pages is not None else None,
            states=cache.states[first:first + len(states)])

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        n = ctx.batch.num_tokens
        left = self.sides[0].forward(x, ctx, self._cache_of(0, cache))
        right = self.sides[1].forward(x, ctx, self._cache_of(1, cache))
        if left.data_ptr() == right.data_ptr():
            raise RuntimeError("two mixers side by side returned the same buffer")
        out = ctx.buffer("side_by_side.out", (n, self.hidden_size))
        kernels.norm_pair_mix(left, right, self.gains[0], self.gains[1], out, n, self.eps, *self.weights)
        return out


register_mixer("side_by_side", SideBySide)
