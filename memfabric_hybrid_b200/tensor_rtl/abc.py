"""Base classes of the resharding layer: a communication task, an executor that runs a list of them, a planner that
orders them. Parity: app/tensorRTL/src/tensor_rtl/api/abc.py of the reference."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import List


@dataclass
class BaseCommTask(ABC):
    """What every task has in common is only that an executor understands it."""


class Executor(ABC):
    def __init__(self):
        self.batch_comm_list: List = []

    @abstractmethod
    def execute(self, tasks: List[BaseCommTask]) -> None:
        """Starts (or runs) the tasks in order."""

    @abstractmethod
    def wait(self) -> None:
        """Returns when every started task is complete."""


class Planner(ABC):
    """Reorders tasks before execution (e.g. to balance links); the default keeps the order. ``topology`` is whatever the
    planner needs to know about the machine. Raises ValueError for a task whose ranks are outside the topology."""

    def __init__(self, topology=None):
        self.topology = topology

    def build_ordered_comm_ops(self, op_list: List[BaseCommTask]) -> List[BaseCommTask]:
        return list(op_list)
