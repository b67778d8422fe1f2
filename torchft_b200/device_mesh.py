"""DeviceMesh glue for hybrid sharding (HSDP) with a fault-tolerant replicate dimension.

Inside a replica group the mesh is an ordinary ``DeviceMesh`` (shard / tensor-parallel
dimensions on fixed process groups).  The replicate dimension spans replica groups
whose number changes at run time, which ``DeviceMesh`` cannot express.  So the real
mesh is built WITHOUT that dimension and ``ManagedDeviceMesh`` presents it virtually:
its process group is a ``ManagedProcessGroup`` and its size is the manager's current
number of participants.

Parity: ``extend_device_mesh``, ``ManagedDeviceMesh`` and ``ft_init_device_mesh`` of the
reference's ``torchft/process_group.py:1057-1331``.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Any, Dict, List, Optional, Tuple, Union

import torch.distributed as dist
from torch.distributed import DeviceMesh, ProcessGroup as BaseProcessGroup, init_device_mesh

if TYPE_CHECKING:
    from torchft_b200.manager import Manager
    from torchft_b200.process_group import ManagedProcessGroup, ProcessGroup


def extend_device_mesh(mesh: DeviceMesh, pg: "ProcessGroup", name: str = "dp", dim: int = 0) -> DeviceMesh:
    """Adds ``pg`` to ``mesh`` as a new dimension ``name`` at position ``dim``.

    DeviceMesh is told the new dimension has extent 1; that is sound as long as all
    scaling by the true world size happens inside ``pg``.
    """
    groups = list(mesh.get_all_groups())
    groups.insert(dim, pg)
    names = list(mesh.mesh_dim_names or [])
    names.insert(dim, name)
    return DeviceMesh.from_group(
        group=groups,
        device_type=mesh.device_type,
        mesh=mesh.mesh.unsqueeze(dim),
        mesh_dim_names=tuple(names),
    )


class ManagedDeviceMesh(DeviceMesh):
    """A mesh whose ``replicate_dim`` is backed by a ``Manager`` instead of a fixed group."""

    # Meshes are pickled by value elsewhere (checkpoints); the process group is not
    # picklable and is re-attached from this per-process singleton.
    replicate_pg_singleton: Optional["ManagedProcessGroup"] = None

    def __init__(
        self,
        mesh: Optional[DeviceMesh],
        mesh_dim_names: Tuple[str, ...],
        replicate_pg: "ManagedProcessGroup",
        replicate_dim: int,
        parent: Optional["ManagedDeviceMesh"],
    ) -> None:
        # DeviceMesh.__init__ is deliberately not called: there is no backing tensor
        # for the virtual dimension.
        if mesh is None and parent is None:
            raise ValueError("ManagedDeviceMesh doesn't support both mesh and parent are None.")
        # DeviceMesh exposes mesh / mesh_dim_names / device_type as read-only properties;
        # they are overridden below and backed by these private fields.
        self._inner_mesh = mesh
        self._dim_names = tuple(mesh_dim_names)
        self.replicate_pg = replicate_pg
        self.replicate_dim = replicate_dim
        self.replicate_dim_name: str = mesh_dim_names[replicate_dim]
        self.parent = parent
        self.flatten_meshes: Dict[str, DeviceMesh] = {}
        inner = mesh if mesh is not None else parent
        assert inner is not None
        self._device_type: str = inner.device_type
        self._flatten_mesh_list: Tuple[DeviceMesh, ...] = tuple()
        self._thread_id: Optional[int] = None

    @property
    def mesh(self) -> Optional[DeviceMesh]:  # type: ignore[override]
        """The real mesh of the dimensions inside the replica group (None for a replicate-only view)."""
        return self._inner_mesh

    @property
    def mesh_dim_names(self) -> Tuple[str, ...]:  # type: ignore[override]
        return self._dim_names

    @property
    def device_type(self) -> str:  # type: ignore[override]
        return self._device_type

    # -- pickling
    def __getstate__(self) -> Dict[str, Any]:
        state = dict(self.__dict__)
        state["replicate_pg"] = None
        return state

    def __setstate__(self, state: Dict[str, Any]) -> None:
        self.__dict__.update(state)
        assert ManagedDeviceMesh.replicate_pg_singleton is not None, "no managed process group in this process"
        self.replicate_pg = ManagedDeviceMesh.replicate_pg_singleton

    # -- helpers
    def _inner(self) -> DeviceMesh:
        assert self.mesh is not None, "this view only holds the replicate dimension"
        return self.mesh

    def _inner_dim(self, dim: int) -> int:
        return dim - 1 if dim > self.replicate_dim else dim

    def _dim_index(self, mesh_dim: Optional[Union[int, str]]) -> int:
        if isinstance(mesh_dim, str):
            return self.mesh_dim_names.index(mesh_dim)
        return 0 if mesh_dim is None else int(mesh_dim)

    def _replicate_size(self) -> int:
        # Before the first quorum there are zero participants; report 1 so callers
        # that divide by the size stay finite.
        n = self.replicate_pg.size()
        return n if n > 0 else 1

    def _replicate_rank(self) -> int:
        return dist.get_rank(self.replicate_pg)

    # -- DeviceMesh interface
    def __getitem__(self, mesh_dim_names: Union[str, Tuple[str, ...]]) -> DeviceMesh:
        if isinstance(mesh_dim_names, str):
            if mesh_dim_names == self.replicate_dim_name:
                return ManagedDeviceMesh(None, (mesh_dim_names,), self.replicate_pg, 0, parent=self)
            if mesh_dim_names in self.flatten_meshes:
                return self.flatten_meshes[mesh_dim_names]
            return self._inner()[mesh_dim_names]
        assert isinstance(mesh_dim_names, tuple)
        if self.replicate_dim_name not in mesh_dim_names:
            return self._inner()[mesh_dim_names]
        rest = tuple(n for n in mesh_dim_names if n != self.replicate_dim_name)
        return ManagedDeviceMesh(
            self._inner()[rest],
            mesh_dim_names,
            self.replicate_pg,
            mesh_dim_names.index(self.replicate_dim_name),
            parent=self,
        )

    def get_group(self, mesh_dim: Optional[Union[int, str]] = None) -> BaseProcessGroup:
        if mesh_dim is None or self._dim_index(mesh_dim) == self.replicate_dim:
            return self.replicate_pg
        return self._inner().get_group(self._inner_dim(self._dim_index(mesh_dim)))

    def _flatten(self, mesh_dim_name: Optional[str] = None, *args: Any, **kwargs: Any) -> DeviceMesh:
        if mesh_dim_name is None:
            raise ValueError("ManagedDeviceMesh._flatten requires `mesh_dim_name`")
        flat = _FlattenDeviceMesh(self)
        owner = self if self.parent is None else self.parent
        owner.flatten_meshes[mesh_dim_name] = flat
        return flat

    def size(self, mesh_dim: Optional[int] = None) -> int:
        if mesh_dim is None:
            inner = 1 if self.mesh is None else self.mesh.size()
            return inner * self._replicate_size()
        if mesh_dim == self.replicate_dim:
            return self._replicate_size()
        return self._inner().size(self._inner_dim(mesh_dim))

    @property
    def ndim(self) -> int:
        return self._inner().ndim + 1

    @property
    def shape(self) -> Tuple[int, ...]:
        dims: List[int] = list(self._inner().shape)
        dims.insert(self.replicate_dim, self.replicate_pg.size())
        return tuple(dims)

    def get_rank(self) -> int:
        return self._inner().get_rank()

    def get_local_rank(self, mesh_dim: Optional[Union[int, str]] = None) -> int:
        if mesh_dim is None:
            if self.mesh is None:
                return self._replicate_rank()
            assert self.replicate_dim == 0, "replicate_dim must be the first one"
            return self.mesh.size() * self._replicate_rank() + self.mesh.get_local_rank()
        dim = self._dim_index(mesh_dim)
        if dim == self.replicate_dim:
            return self._replicate_rank()
        return self._inner().get_local_rank(self._inner_dim(dim))

    def get_coordinate(self) -> Optional[List[int]]:
        """Coordinates of this rank along every dimension, the virtual one included."""
        inner = self._inner().get_coordinate()
        if not inner:
            return inner
        coord = list(inner)
        coord.insert(self.replicate_dim, self._replicate_rank())
        return coord

    @property
    def _coordinate_on_dim(self) -> Optional[List[int]]:
        # DTensor asks the mesh whether this rank is part of it through this private field
        return self.get_coordinate()

    def get_all_groups(self) -> List[BaseProcessGroup]:
        raise NotImplementedError

    def __repr__(self) -> str:
        return f"ManagedDeviceMesh(mesh={self.mesh}, dims={self.mesh_dim_names}, replicate_dim={self.replicate_dim})"

    def __hash__(self) -> int:
        return hash((id(self.replicate_pg), self.mesh_dim_names, self.replicate_dim, hash(self.mesh) if self.mesh is not None else 0))

    def __eq__(self, other: object) -> bool:
        if not isinstance(other, ManagedDeviceMesh):
            return False
        return (
            self.replicate_pg is other.replicate_pg
            and self.mesh_dim_names == other.mesh_dim_names
            and self.replicate_dim == other.replicate_dim
            and self.mesh == other.mesh
        )


class _FlattenDeviceMesh(DeviceMesh):
    """Result of flattening a managed mesh: only total size and flat local rank exist."""

    def __init__(self, managed_mesh: ManagedDeviceMesh) -> None:
        self.managed_mesh = managed_mesh

    def __getitem__(self, mesh_dim_names: Union[str, Tuple[str, ...]]) -> DeviceMesh:
        raise NotImplementedError

    def get_group(self, mesh_dim: Optional[Union[int, str]] = None) -> BaseProcessGroup:
        raise NotImplementedError

    def _flatten(self, mesh_dim_name: Optional[str] = None, *args: Any, **kwargs: Any) -> DeviceMesh:
        raise NotImplementedError

    def size(self, mesh_dim: Optional[int] = None) -> int:
        assert mesh_dim is None
        return self.managed_mesh.size()

    @property
    def ndim(self) -> int:
        raise NotImplementedError

    @property
    def shape(self) -> Tuple[int, ...]:
        raise NotImplementedError

    def get_rank(self) -> int:
        raise NotImplementedError

    def get_local_rank(self, mesh_dim: Optional[Union[int, str]] = None) -> int:
        assert mesh_dim is None
        return self.managed_mesh.get_local_rank()

    def get_all_groups(self) -> List[BaseProcessGroup]:
        raise NotImplementedError

    def __hash__(self) -> int:
        return hash(("flat", id(self.managed_mesh)))

    def __eq__(self, other: object) -> bool:
        return isinstance(other, _FlattenDeviceMesh) and other.managed_mesh is self.managed_mesh


def ft_init_device_mesh(
    *,
    device_type: str,
    mesh_shape: Tuple[int, ...],
    mesh_dim_names: Tuple[str, ...],
    replicate_dim: int,
    manager: "Manager",
) -> ManagedDeviceMesh:
    """Builds the in-group mesh (all dimensions but ``replicate_dim``) and wraps it.

    ``mesh_shape[replicate_dim]`` is ignored: that extent is whatever the quorum says.
    """
    from torchft_b200.process_group import ManagedProcessGroup

    inner_shape = list(mesh_shape)
    inner_shape.pop(replicate_dim)
    inner_names = list(mesh_dim_names)
    inner_names.pop(replicate_dim)
    mesh = init_device_mesh(device_type, mesh_shape=tuple(inner_shape), mesh_dim_names=tuple(inner_names))

    replicate_pg = ManagedProcessGroup(manager)
    replicate_pg.register(mesh_dim_names[replicate_dim])
    ManagedDeviceMesh.replicate_pg_singleton = replicate_pg

    return ManagedDeviceMesh(
        mesh=mesh,
        mesh_dim_names=mesh_dim_names,
        replicate_pg=replicate_pg,
        replicate_dim=replicate_dim,
        parent=None,
    )
