"""Architectures this framework serves. Importing the package registers them."""

from . import diderax, fegilix, gasavik, guzovik, qwen3  # noqa: F401  (registers Diderax, Fegilix, Gasavik, Guzovik and Qwen3ForCausalLM)
from .diderax import DideraxConfig
from .fegilix import FegilixConfig
from .gasavik import GasavikConfig
from .guzovik import GuzovikConfig
from .qwen3 import Qwen3Config

__all__ = ["DideraxConfig", "FegilixConfig", "GasavikConfig", "GuzovikConfig", "Qwen3Config"]
