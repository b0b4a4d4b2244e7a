"""Placeholder kept for import compatibility (the reference ships an empty
``ScheduleSolver`` class, pfeife/schedule/solver.py:1-9)."""


class ScheduleSolver:
    pass
