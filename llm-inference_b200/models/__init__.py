"""Architectures this engine knows; importing the package registers them."""

from . import gunedra, lerorax, qwen2, tunadra, zetizen  # noqa: F401
