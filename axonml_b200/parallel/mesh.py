"""Device mesh: names the dimensions of a multi-way parallel layout and owns one process group per
dimension.

    mesh = DeviceMesh(world, {"pp": 2, "tp": 4})     # 8 ranks; the LAST dimension varies fastest
    mesh.group("tp")                                   # ranks that share this rank's pp coordinate
    mesh.coord("pp"), mesh.size("tp")

Rank r has coordinates ``unravel(r, sizes)`` in row-major order, so with ``{"pp": 2, "tp": 4}``
ranks 0..3 form the first tensor-parallel group (one pipeline stage) and ranks {0, 4} a pipeline
group: neighbouring ranks (same NVSwitch box in a larger job) share the dimension that talks the
most.  Every rank creates every group - the process-group rendezvous requires it - and keeps its own.

The reference stores a rank list per group but its collectives ignore it
(crates/axonml-distributed/src/process_group.rs:34-36, :86-90); here sub-groups are real."""
from __future__ import annotations

from .process_group import ProcessGroup, World


class DeviceMesh:
    def __init__(self, world: World, shape: dict):
        self.world = world
        self.names = list(shape)
        self.sizes = [int(shape[n]) for n in self.names]
        total = 1
        for s in self.sizes:
            total *= s
        if total != world.world_size():
            raise ValueError(f"mesh {shape} needs {total} ranks, the world has {world.world_size()}")
        self.rank = world.rank()
        self._coords = self._unravel(self.rank)
        self._groups: dict[str, ProcessGroup] = {}
        for d, name in enumerate(self.names):
            mine = None
            for base in self._bases(d):
                ranks = [base + i * self._stride(d) for i in range(self.sizes[d])]
                g = world.new_group(ranks)
                if self.rank in ranks:
                    mine = g
            self._groups[name] = mine

    def _stride(self, d: int) -> int:
        s = 1
        for x in self.sizes[d + 1:]:
            s *= x
        return s

    def _unravel(self, r: int) -> list:
        out = []
        for d in range(len(self.sizes)):
            st = self._stride(d)
            out.append(r // st % self.sizes[d])
        return out

    def _bases(self, d: int):
        """First rank of every group along dimension ``d``."""
        st, n = self._stride(d), self.sizes[d]
        total = 1
        for s in self.sizes:
            total *= s
        return [r for r in range(total) if r // st % n == 0]

    def group(self, name: str) -> ProcessGroup: return self._groups[name]
    def coord(self, name: str) -> int: return self._coords[self.names.index(name)]
    def size(self, name: str) -> int: return self.sizes[self.names.index(name)]
    def coords(self) -> dict: return dict(zip(self.names, self._coords))

    def ranks(self, name: str) -> list:
        d = self.names.index(name)
        base = self.rank - self._coords[d] * self._stride(d)
        return [base + i * self._stride(d) for i in range(self.sizes[d])]
