"""sllm_b200: a Blackwell-native (sm_100a) LLM inference engine with the capabilities of sLLM."""
__version__ = "0.1.0"
