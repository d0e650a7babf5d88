from .arena import CosineSchedule, FlatArena, FlatSGD

__all__ = ["FlatArena", "FlatSGD", "CosineSchedule"]
