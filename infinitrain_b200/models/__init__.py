from .gpt2 import GPT2, gpt2_config
from .llama3 import LLaMA3, llama3_config
