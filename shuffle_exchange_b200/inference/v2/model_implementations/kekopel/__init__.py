from .policy import KekopelPolicy  # noqa: F401
