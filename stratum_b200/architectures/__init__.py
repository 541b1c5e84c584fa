from . import dabodra, llama, nibelorn  # noqa: F401  (registers the architectures)
