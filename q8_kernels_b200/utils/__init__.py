from . import convert_weights  # noqa: F401
