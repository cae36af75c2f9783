"""smcsd_b200: a Blackwell-native Sequential-Monte-Carlo speculative-decoding engine."""
from .config import EngineArgs
from .engine import SMCEngine

__all__ = ["SMCEngine", "EngineArgs"]
__version__ = "0.1.0"
