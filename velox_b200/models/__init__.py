"""Built-in architectures.  Importing this package registers them."""
from . import lizizen, peratar, qwen2, redalix  # noqa: F401
