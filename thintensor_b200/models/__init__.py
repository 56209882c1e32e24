"""Built-in architectures.  Importing this package registers them."""
from . import famalorn, kerepel, llama, neruzen, sogidra  # noqa: F401
