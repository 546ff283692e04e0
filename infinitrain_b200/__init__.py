"""infinitrain_b200: a Blackwell-native (sm_100a) LLM training framework."""
__version__ = "0.1.0"
