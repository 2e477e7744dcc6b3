"""Schedule parameters and the tile database (the reference's ``lighthouse.schedule``)."""

from .parameters import ScheduleParameters
from .tile_selector import CudaTileSelector, TILE_WIDTHS

__all__ = ["ScheduleParameters", "CudaTileSelector", "TILE_WIDTHS"]
