"""Models.  Importing the package registers the built-in architectures."""
from . import fosepel, geponex, qwen2, sisetar, vegilix  # noqa: F401
from .base import DecoderModel
