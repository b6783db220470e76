from . import layer, utils  # noqa: F401
