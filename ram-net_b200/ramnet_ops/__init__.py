from . import _C  # noqa: F401
