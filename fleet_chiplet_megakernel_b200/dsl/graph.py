"""Graph session and tensor wrapper of the DSL (python/mirage/mpk/dsl/graph.py of the reference)."""
import torch

from ..persistent_kernel import bfloat16, convert_torch_type_to_dtype


class Tensor:
    """A DTensor of the PersistentKernel with its name and the graph it belongs to."""

    def __init__(self, dtensor, name, graph):
        self.dt, self.name, self.graph = dtensor, name, graph

    def dim(self, i):
        return self.dt.dim(i)

    @property
    def num_dims(self):
        return self.dt.num_dims

    @property
    def shape(self):
        return tuple(self.dt.dims)

    def __repr__(self):
        return f"Tensor({self.name}, shape={self.shape})"


class Graph:
    """``g = Graph(mpk)``; ``g.input(torch_tensor, name)``, ``g.intermediate(dims, name=...)``,
    ``g.shuffle_inputs([...], num_groups, name)``, then op functions from ``dsl.ops``."""

    def __init__(self, mpk):
        self.mpk = mpk
        self._scratch = {}
        self._next = 0

    def input(self, torch_tensor, name):
        return Tensor(self.mpk.attach_input(torch_tensor=torch_tensor, name=name), name, self)

    def intermediate(self, dims, dtype=bfloat16, name=None):
        name = name or f"_intermediate_{self._next}"
        self._next += 1
        return Tensor(self.mpk.new_tensor(dims=tuple(dims), dtype=dtype, name=name), name, self)

    def _unwrap(self, ts):
        return [t.dt if isinstance(t, Tensor) else t for t in ts]

    def shuffle_inputs(self, dtensors, num_groups, name):
        return Tensor(self.mpk.shuffle_tensors(inputs=self._unwrap(dtensors), shuffled_dim=0, num_groups=num_groups,
                                               name=name), name, self)

    def fuse_inputs(self, dtensors, name):
        return Tensor(self.mpk.fuse_tensors(inputs=self._unwrap(dtensors), fused_dim=0, num_groups=1, name=name), name, self)

    # The reference's gang kernels need caller-provided workspaces and done counters.  Here the runtime owns
    # its split-k scratch, so these are runtime-owned placeholders that the layers accept and never touch
    # (one per shape, shared between layers like the reference's pool).
    def get_workspace(self, rows, cols, dtype=torch.float32, hint="ws"):
        key = ("ws", rows, cols, str(dtype))
        if key not in self._scratch:
            self._scratch[key] = self.mpk.new_tensor(dims=(rows, cols), dtype=convert_torch_type_to_dtype(dtype),
                                                     name=f"_dsl_{hint}_{len(self._scratch)}")
        return self._scratch[key]

    def get_counter(self, n_blocks, hint="dc"):
        key = ("dc", n_blocks)
        if key not in self._scratch:
            self._scratch[key] = self.mpk.new_tensor(dims=(n_blocks, 1), dtype=convert_torch_type_to_dtype(torch.int32),
                                                     name=f"_dsl_{hint}_{len(self._scratch)}")
        return self._scratch[key]
