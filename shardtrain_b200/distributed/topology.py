"""F x T rank mesh arithmetic (pure Python).

Rank r sits at (fsdp, tp) = divmod(r, T): the TP coordinate varies fastest, so a TP/SP group is
T consecutive ranks and an FSDP group strides by T.  Same mapping as the reference
(`src/sharded_runtime/distributed/topology.py:26-65`), so rank files and logs line up.
"""

from __future__ import annotations

from dataclasses import dataclass

GROUP_ROLES = ("tp", "fsdp", "tp_grad", "fsdp_grad")


@dataclass(frozen=True)
class RankCoordinate:
    fsdp: int
    tp: int


def _positive_int(name: str, value: object) -> None:
    if type(value) is not int or value <= 0:
        raise ValueError(f"{name} must be a positive integer")


@dataclass(frozen=True)
class Topology:
    fsdp_degree: int
    tp_degree: int

    def __post_init__(self) -> None:
        _positive_int("fsdp_degree", self.fsdp_degree)
        _positive_int("tp_degree", self.tp_degree)

    @property
    def world_size(self) -> int:
        return self.fsdp_degree * self.tp_degree

    def coordinate(self, rank: int) -> RankCoordinate:
        if type(rank) is not int or not 0 <= rank < self.world_size:
            raise ValueError(f"rank must be in [0, {self.world_size}); got {rank!r}")
        f, t = divmod(rank, self.tp_degree)
        return RankCoordinate(f, t)

    def rank(self, fsdp: int, tp: int) -> int:
        if type(fsdp) is not int or not 0 <= fsdp < self.fsdp_degree:
            raise ValueError(f"Invalid FSDP coordinate: {fsdp!r}")
        if type(tp) is not int or not 0 <= tp < self.tp_degree:
            raise ValueError(f"Invalid TP coordinate: {tp!r}")
        return fsdp * self.tp_degree + tp

    @property
    def tp_groups(self) -> tuple[tuple[int, ...], ...]:
        T = self.tp_degree
        return tuple(tuple(range(f * T, (f + 1) * T)) for f in range(self.fsdp_degree))

    @property
    def fsdp_groups(self) -> tuple[tuple[int, ...], ...]:
        T = self.tp_degree
        return tuple(tuple(range(t, self.world_size, T)) for t in range(T))

    @property
    def creation_order(self) -> tuple[tuple[str, tuple[int, ...]], ...]:
        """Every (role, members) communicator, in the order every rank must create them.

        The gradient roles repeat the memberships of `tp` and `fsdp` on purpose: a separate
        communicator keeps gradient reduction from ordering parameter gathers or activation
        collectives.
        """
        by_role = {
            "tp": self.tp_groups,
            "fsdp": self.fsdp_groups,
            "tp_grad": self.tp_groups,
            "fsdp_grad": self.fsdp_groups,
        }
        return tuple((role, members) for role in GROUP_ROLES for members in by_role[role])

    def groups_for_rank(self, rank: int) -> dict[str, tuple[int, ...]]:
        c = self.coordinate(rank)
        tp, fsdp = self.tp_groups[c.fsdp], self.fsdp_groups[c.tp]
        return {"tp": tp, "fsdp": fsdp, "tp_grad": tp, "fsdp_grad": fsdp}
