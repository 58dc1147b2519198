"""B200-native quantized LLM inference engine."""
__version__ = "0.1.0"
