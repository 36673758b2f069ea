"""Annotations for task signatures in the DSL (python/mirage/mpk/dsl/types.py of the reference).

They document how an operand is split and are never enforced: ``Tile[M, K]`` an operand every
worker sees whole, ``Partition[N // 8, K]`` one that is cut between groups of workers (XCDs in the
reference, SMs / dies here), ``Chunk`` a chunk of the KV cache."""


class _Shape:
    def __class_getitem__(cls, dims):
        return cls(*dims) if isinstance(dims, tuple) else cls(dims)

    def __init__(self, *dims):
        self.dims = dims

    def __repr__(self):
        return f"{type(self).__name__}[{', '.join(str(d) for d in self.dims)}]"


class Tile(_Shape):
    """An operand that is broadcast, not partitioned (activations)."""


class Partition(_Shape):
    """An operand cut between worker groups (weight rows)."""


class Chunk:
    """A chunk of the KV cache (one per worker group for cache affinity)."""

    def __repr__(self):
        return "Chunk"
