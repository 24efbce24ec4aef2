from .symm import SymmetricArena, symmetric_memory_available  # noqa: F401
