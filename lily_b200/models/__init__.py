"""Architectures this package ships; importing the package registers them."""

from lily_b200.models import dense_decoder  # noqa: F401
