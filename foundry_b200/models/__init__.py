"""Built-in architectures; importing this package registers them."""
from . import llama, rupotar, vikarax, vonulorn  # noqa: F401
