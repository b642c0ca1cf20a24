"""Architectures (as data) and the generic model.  Importing registers the built-in ones."""
from .model import Model
from . import mqa_gpt, munevik, mizupel, mokalorn, dabilorn  # noqa: F401  (registration)
