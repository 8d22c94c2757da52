"""nanochat-b200: a Blackwell-native (sm_100a) full-stack LLM training / inference framework."""

__version__ = "0.1.0"
