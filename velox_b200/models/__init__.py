"""Built-in architectures.  Importing this package registers them."""
from . import lizizen, mamivik, peratar, qwen2, redalix  # noqa: F401
