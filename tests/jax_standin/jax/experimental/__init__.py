from . import pallas  # noqa: F401
