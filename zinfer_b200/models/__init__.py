"""Architectures.  Importing this package registers every architecture the library has."""
from .model import LayerCall, Model
from . import lfm2  # noqa: F401  (registers Lfm2ForCausalLM)
