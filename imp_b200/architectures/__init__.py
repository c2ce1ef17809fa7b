"""Built-in architectures; importing this package registers them."""
from . import qwen3  # noqa: F401
