from .policy import FomalixPolicy  # noqa: F401
