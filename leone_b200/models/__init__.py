"""Built-in architectures.  Importing this package registers them."""
from . import qwen3  # noqa: F401
