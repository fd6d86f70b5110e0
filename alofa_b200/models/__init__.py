"""Built-in architectures.  Importing this package registers them."""
from . import darolix, kotutar, qwen2  # noqa: F401
