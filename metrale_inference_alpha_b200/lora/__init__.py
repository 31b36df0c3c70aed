from .manager import LoraAdapter, LoraManager  # noqa: F401
