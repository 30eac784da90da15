"""Two mixers side by side as one mixer: both read the same input and the result is
scale_a * a(h) + scale_b * b(h).  The children are any registered mixers (``left`` and ``right``
are their :class:`~pretrained_rstr_b200.config.base.PartSpec`s); each gets its constant as
``out_scale``, applied in 32-bit before its output projection, and adds its projection to the
stream itself.  At most one child may keep keys and values (the layer has one cache); the
children's states are declared together (their names must differ).  Where the first child keeps
its projections in one fused product and offers room in it (``fuse_input_rows``) and the second
child can take its own from a host (``takes_input_host``), the second child's projections ride
in the first child's product: one product a layer reads the stream for both (``input_host`` is
offered to every second child; one that keeps a product of its own over another input ignores
it).  ``share_product`` False keeps the products apart."""
from __future__ import annotations

from .interfaces import LayerCache, Mixer
from .registry import build_part, register_part


class SideBySide(Mixer):
    can_overwrite = True

    def __init__(self, p: dict, store, runtime):
        self.children = []
        for side in ("left", "right"):
            spec = p[side]
            extra = {"out_scale": float(p.get(side + "_scale", 1.0))}
            if self.children and hasattr(self.children[0], "fuse_input_rows") and \
                    hasattr(self.children[0], "fused_product") and p.get("share_product", True):
                extra["input_host"] = self.children[0]
            scaled = type(spec)(spec.kind, {**spec.params, **extra})
            self.children.append(build_part("mixer", scaled, store, runtime))
        if sum(c.kv_spec() is not None for c in self.children) > 1:
            raise ValueError("side_by_side: only one of the two mixers may keep keys and values")
        names = [s.name for c in self.children for s in c.state_specs()]
        if len(set(names)) != len(names):
            raise ValueError("side_by_side: the two mixers declare state of the same name")
        for c in self.children:
            if not getattr(c, "can_overwrite", False):
                raise ValueError(f"side_by_side: {type(c).__name__} cannot start a sum")

    @property
    def graph_safe(self) -> bool:
        return all(getattr(c, "graph_safe", False) for c in self.children)

    def kv_spec(self):
        for c in self.children:
            if c.kv_spec() is not None:
                return c.kv_spec()
        return None

    def state_specs(self):
        return [s for c in self.children for s in c.state_specs()]

    def work_planners(self) -> list:
        return [w for c in self.children for w in c.work_planners()]

    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        first, second = self.children
        first.forward(ctx, h, x, cache, accumulate=accumulate)
        second.forward(ctx, h, x, cache, accumulate=True)


register_part("mixer", "side_by_side", lambda p, store, rt: SideBySide(p, store, rt))
