from . import state  # noqa: F401
