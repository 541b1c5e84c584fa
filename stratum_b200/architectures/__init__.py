from . import llama, nibelorn  # noqa: F401  (registers the architectures)
