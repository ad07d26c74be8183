"""Declarative benchmark recipes."""
from .recipe import Recipe, run_recipe  # noqa: F401
