from .spec import Condition, Field, InputSpec, unit_range

__all__ = ["Condition", "Field", "InputSpec", "unit_range"]
