"""Architectures this framework serves. Importing the package registers them."""

from . import fegilix, gasavik, guzovik, qwen3  # noqa: F401  (registers Fegilix, Gasavik, Guzovik and Qwen3ForCausalLM)
from .fegilix import FegilixConfig
from .gasavik import GasavikConfig
from .guzovik import GuzovikConfig
from .qwen3 import Qwen3Config

__all__ = ["FegilixConfig", "GasavikConfig", "GuzovikConfig", "Qwen3Config"]
