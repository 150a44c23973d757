from .quantizer import Bitween  # noqa: F401
