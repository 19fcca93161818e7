"""Architectures.  Importing this package registers them."""

from . import dopudra, llama, pudulorn, zadurax  # noqa: F401
