"""Blackwell-native Dual-Mod attention framework."""
from .config import DualModConfig, TrainConfig, preset

__all__ = ["DualModConfig", "TrainConfig", "preset"]
__version__ = "0.1.0"
