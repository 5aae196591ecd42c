"""Architectures this package ships; importing the package registers them."""

from lily_b200.models import dense_decoder, godotar, gotivik, kinanex, zirurax  # noqa: F401
