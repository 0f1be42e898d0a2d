"""Model-side helpers: dtype casting, gradient release, timing."""

from .cast import cast_model
from .gradient_release import GradientReleaseHandle, enable_gradient_release

__all__ = ["cast_model", "enable_gradient_release", "GradientReleaseHandle"]
