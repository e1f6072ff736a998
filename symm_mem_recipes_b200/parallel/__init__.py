from . import symm_mem  # noqa: F401
