"""``@task``, ``@distribute`` and ``@affinity``: scheduling metadata on op functions
(python/mirage/mpk/dsl/decorators.py of the reference).

The decorators only attach a ``_fleet_meta`` dict to the function; ``dsl.ops.linear`` reads it
(through ``strategy=`` passed by the decorated function, or ``strategy_from_meta``) to pick how the
layer is recorded.  The reference's levels name MI300 scopes (warp / cu / xcd); on B200 the scopes are
warp / sm / cluster / gpu, and the reference's names stay accepted: "cu" means "sm", "xcd" (a cache
domain the workers of one chiplet share) means "gpu", because all 148 SMs share one coherent L2."""
from functools import wraps

_LEVELS = {"warp": "warp", "cu": "sm", "sm": "sm", "cluster": "cluster", "xcd": "gpu", "die": "gpu", "gpu": "gpu",
           "auto": "auto"}


def parse_budget(budget):
    """'4MB' / '512KB' / '100B' / a number -> bytes (None stays None)."""
    if budget is None or isinstance(budget, (int, float)):
        return None if budget is None else int(budget)
    s = str(budget).strip().upper()
    for suffix, mul in (("MB", 1 << 20), ("KB", 1 << 10), ("B", 1)):
        if s.endswith(suffix):
            return int(float(s[: -len(suffix)]) * mul)
    return int(s)


def get_meta(fn):
    return getattr(fn, "_fleet_meta", {})


class task:
    """level: "warp" | "sm" ("cu") | "cluster" | "gpu" ("xcd") | "auto";  tiling: "cooperative_3d" |
    "split_k" | "auto";  l2_budget: bytes or a string like "4MB" (how much of L2 the op's weights may hold)."""

    def __init__(self, level="auto", tiling="auto", l2_budget=None):
        if level not in _LEVELS:
            raise ValueError(f"unknown task level {level!r}")
        self.level, self.tiling, self.l2_budget = level, tiling, l2_budget

    def __call__(self, fn):
        meta = dict(get_meta(fn))
        meta.update(level=self.level, scope=_LEVELS[self.level], tiling=self.tiling, l2_budget=parse_budget(self.l2_budget))
        fn._fleet_meta = meta
        return fn

    def __repr__(self):
        return f"@task(level={self.level!r}, tiling={self.tiling!r}, l2_budget={self.l2_budget!r})"


class distribute:
    """Partition the op's weight along ``dim`` between ``num_xcds`` worker groups.  The runtime always
    deals weight rows (or row-block x k tiles) over all SMs itself; the numbers are kept as metadata."""

    def __init__(self, dim=0, num_xcds=8):
        self.dim, self.num_xcds = dim, num_xcds

    def __call__(self, fn):
        @wraps(fn)
        def wrapper(*args, **kwargs):
            return fn(*args, **kwargs)

        meta = dict(get_meta(fn))
        meta["partition"] = {"dim": self.dim, "num_xcds": self.num_xcds}
        wrapper._fleet_meta = meta
        return wrapper

    def __repr__(self):
        return f"@distribute(dim={self.dim}, num_xcds={self.num_xcds})"


class affinity:
    """placement="inherit_xcd": run where the producer of the input ran.  A hint (as in the reference): every
    CTA of the persistent kernel walks the same static program, so consumer and producer shares of an op
    already sit on the same SMs from one iteration to the next."""

    def __init__(self, placement="inherit_xcd"):
        self.placement = placement

    def __call__(self, fn):
        meta = dict(get_meta(fn))
        meta["placement"] = self.placement
        fn._fleet_meta = meta
        return fn

    def __repr__(self):
        return f"@affinity(placement={self.placement!r})"


def strategy_from_meta(meta):
    """Decorator metadata -> a strategy name for ``ops.linear`` ("auto" lets the cost model choose).
    warp / sm tasks are plain layers; a gpu- ("xcd"-) level task asks for the cooperative forms, whose
    tiling arguments the runtime treats as hints."""
    scope = meta.get("scope", _LEVELS.get(meta.get("level", "auto"), "auto"))
    tiling = meta.get("tiling", "auto")
    if scope in ("warp", "sm"):
        return "standard"
    if scope in ("gpu", "cluster"):
        if tiling == "split_k":
            return "gang_splitk"
        return "gang"
    return "auto"
