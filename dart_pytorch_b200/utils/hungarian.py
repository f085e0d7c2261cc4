"""Minimum-cost assignment on a square integer cost matrix (reference: lib/core/utils/hungarian_algorithm.dart).

``HungarianAlgorithm(costs).get_assignment()[agent] = task``.  Rectangular problems are padded by the caller with a
large sentinel cost, as in the DETR-style matching demos.  The solver is the O(n^3) shortest-augmenting-path form with
row / column potentials (exact for integers, ties broken towards the lowest column index).
"""
from __future__ import annotations

from typing import List, Sequence


class HungarianAlgorithm:
    def __init__(self, cost_matrix: Sequence[Sequence[int]]):
        n = len(cost_matrix)
        for row in cost_matrix:
            if len(row) != n:
                raise ValueError("HungarianAlgorithm: cost matrix must be square")
        self._n = n
        self._cost = [[int(v) for v in row] for row in cost_matrix]
        self._assignment: List[int] = []

    def get_assignment(self) -> List[int]:
        if self._assignment or self._n == 0:
            return list(self._assignment)
        n, cost = self._n, self._cost
        INF = float("inf")
        u = [0] * (n + 1)          # row potentials
        v = [0] * (n + 1)          # column potentials
        match = [0] * (n + 1)      # match[col] = row (1-based), 0 = free
        way = [0] * (n + 1)
        for i in range(1, n + 1):
            match[0] = i
            j0 = 0
            minv = [INF] * (n + 1)
            used = [False] * (n + 1)
            while True:
                used[j0] = True
                i0, delta, j1 = match[j0], INF, 0
                row = cost[i0 - 1]
                for j in range(1, n + 1):
                    if used[j]:
                        continue
                    cur = row[j - 1] - u[i0] - v[j]
                    if cur < minv[j]:
                        minv[j], way[j] = cur, j0
                    if minv[j] < delta:
                        delta, j1 = minv[j], j
                for j in range(n + 1):
                    if used[j]:
                        u[match[j]] += delta
                        v[j] -= delta
                    else:
                        minv[j] -= delta
                j0 = j1
                if match[j0] == 0:
                    break
            while j0:
                j1 = way[j0]
                match[j0] = match[j1]
                j0 = j1
        out = [0] * n
        for j in range(1, n + 1):
            out[match[j] - 1] = j - 1
        self._assignment = out
        return list(out)

    getAssignment = get_assignment

    def total_cost(self) -> int:
        a = self.get_assignment()
        return sum(self._cost[i][a[i]] for i in range(self._n))
