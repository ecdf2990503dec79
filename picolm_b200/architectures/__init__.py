"""Architectures known to the library.  Importing this package registers them;
a new one is a new module here that calls `register_architecture`."""
from . import fupapel, kunulorn, llama, potuzen, tebasun  # noqa: F401
