"""Built-in architectures.  Importing this package registers them."""
from . import kotutar, qwen2  # noqa: F401
