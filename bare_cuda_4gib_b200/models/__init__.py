"""Architectures.  Importing this package registers them."""

from . import dopudra, gurolix, llama, pudulorn, zadurax  # noqa: F401
