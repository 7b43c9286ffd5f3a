"""Rank -> parallel-group arithmetic for one node, with the semantics of the reference's
``Mapping`` (tensorrt_llm/mapping.py:114-258 of TensorRT-LLM): ranks are laid out tp-fastest, then
cp, then pp. Only what the tensor-parallel linear layers need is kept (no MoE / auto-parallel)."""
from __future__ import annotations

from typing import List


class Mapping:
    def __init__(self, world_size: int = 1, rank: int = 0, gpus_per_node: int = 8, *, tp_size: int = 1,
                 pp_size: int = 1, cp_size: int = 1):
        if tp_size * pp_size * cp_size != world_size:
            raise ValueError(f"world_size must equal to tp_size * pp_size * cp_size, but got {world_size} != "
                             f"{tp_size} * {pp_size} * {cp_size}.")
        if not isinstance(rank, int) or rank < 0 or rank >= world_size:
            raise ValueError(f"Rank should be an integer between 0 and {world_size - 1}, but got {rank}.")
        self.world_size, self.rank, self.gpus_per_node = world_size, rank, gpus_per_node
        self.tp_size, self.pp_size, self.cp_size = tp_size, pp_size, cp_size
        block = tp_size * cp_size  # ranks of one pipeline stage
        self.tp_groups: List[List[int]] = [
            [p * block + c * tp_size + t for t in range(tp_size)] for p in range(pp_size) for c in range(cp_size)]
        self.cp_groups: List[List[int]] = [
            [p * block + c * tp_size + t for c in range(cp_size)] for p in range(pp_size) for t in range(tp_size)]
        self.pp_groups: List[List[int]] = [[p * block + i for p in range(pp_size)] for i in range(block)]

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp_size

    @property
    def cp_rank(self) -> int:
        return self.rank % (self.tp_size * self.cp_size) // self.tp_size

    @property
    def pp_rank(self) -> int:
        return self.rank // (self.tp_size * self.cp_size)

    @property
    def tp_group(self) -> List[int]:
        return self.tp_groups[self.pp_rank * self.cp_size + self.cp_rank]

    @property
    def cp_group(self) -> List[int]:
        return self.cp_groups[self.pp_rank * self.tp_size + self.tp_rank]

    @property
    def pp_group(self) -> List[int]:
        return self.pp_groups[self.cp_rank * self.tp_size + self.tp_rank]

    def has_tp(self) -> bool:
        return self.tp_size > 1

    @property
    def local_rank(self) -> int:
        return self.rank % self.gpus_per_node

    def is_first_pp_rank(self) -> bool:
        return self.pp_rank == 0

    def is_last_pp_rank(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    def __eq__(self, other):
        if not isinstance(other, Mapping):
            return NotImplemented
        return (self.world_size, self.rank, self.gpus_per_node, self.tp_size, self.pp_size, self.cp_size) == (
            other.world_size, other.rank, other.gpus_per_node, other.tp_size, other.pp_size, other.cp_size)

    def __hash__(self):
        return hash((self.world_size, self.rank, self.gpus_per_node, self.tp_size, self.pp_size, self.cp_size))
