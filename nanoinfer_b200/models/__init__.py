from .model import Model
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = ["Model", "ModelSpec", "LayerSpec", "PartSpec", "ScheduleEntry"]
