"""Built-in architectures.  Importing this package registers them."""
from . import famalorn, llama, neruzen, sogidra  # noqa: F401
