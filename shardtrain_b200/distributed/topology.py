"""F x T rank mesh arithmetic (pure Python).

Rank r sits at (fsdp, tp) = divmod(r, T): the TP coordinate varies fastest, so a TP/SP group is
T consecutive ranks and an FSDP group strides by T.  Same mapping as the reference
(`src/sharded_runtime/distributed/topology.py:26-65`), so rank files and logs line up.

The mesh is described by its two axes; a communicator role names the axis it runs along, and
every group is "all ranks that differ only in that axis' coordinate".
"""

from __future__ import annotations

from dataclasses import dataclass

AXES = ("fsdp", "tp")                      # slowest to fastest varying coordinate
# role -> axis.  The gradient roles repeat the memberships of `tp` and `fsdp` on purpose: a
# separate communicator keeps gradient reduction from ordering parameter gathers or activation
# collectives.
ROLE_AXIS = {"tp": "tp", "fsdp": "fsdp", "tp_grad": "tp", "fsdp_grad": "fsdp"}
GROUP_ROLES = tuple(ROLE_AXIS)


@dataclass(frozen=True)
class RankCoordinate:
    fsdp: int
    tp: int


@dataclass(frozen=True)
class Topology:
    fsdp_degree: int
    tp_degree: int

    def __post_init__(self) -> None:
        for axis in AXES:
            degree = self.degree(axis)
            if type(degree) is not int or degree <= 0:
                raise ValueError(f"{axis}_degree must be a positive integer")

    def degree(self, axis: str) -> int:
        return getattr(self, f"{axis}_degree")

    @property
    def world_size(self) -> int:
        return self.fsdp_degree * self.tp_degree

    def coordinate(self, rank: int) -> RankCoordinate:
        if type(rank) is not int or not 0 <= rank < self.world_size:
            raise ValueError(f"rank must be in [0, {self.world_size}); got {rank!r}")
        return RankCoordinate(*divmod(rank, self.tp_degree))

    def rank(self, fsdp: int, tp: int) -> int:
        for axis, value in (("fsdp", fsdp), ("tp", tp)):
            if type(value) is not int or not 0 <= value < self.degree(axis):
                raise ValueError(f"Invalid {axis.upper()} coordinate: {value!r}")
        return fsdp * self.tp_degree + tp

    def groups_along(self, axis: str) -> tuple[tuple[int, ...], ...]:
        """The communicators of one axis: one per value of the other axis, members in the order
        of the axis' own coordinate."""
        other = next(a for a in AXES if a != axis)
        return tuple(
            tuple(self.rank(**{axis: moving, other: fixed}) for moving in range(self.degree(axis)))
            for fixed in range(self.degree(other)))

    @property
    def tp_groups(self) -> tuple[tuple[int, ...], ...]:
        return self.groups_along("tp")

    @property
    def fsdp_groups(self) -> tuple[tuple[int, ...], ...]:
        return self.groups_along("fsdp")

    @property
    def creation_order(self) -> tuple[tuple[str, tuple[int, ...]], ...]:
        """Every (role, members) communicator, in the order every rank must create them."""
        return tuple((role, members) for role in GROUP_ROLES
                     for members in self.groups_along(ROLE_AXIS[role]))

    def groups_for_rank(self, rank: int) -> dict[str, tuple[int, ...]]:
        self.coordinate(rank)                      # validates the rank
        mine = {axis: next(g for g in self.groups_along(axis) if rank in g) for axis in AXES}
        return {role: mine[axis] for role, axis in ROLE_AXIS.items()}
