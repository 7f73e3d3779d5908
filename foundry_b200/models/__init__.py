"""Built-in architectures; importing this package registers them."""
from . import kutepel, llama, rupotar, vikarax, vonulorn  # noqa: F401
