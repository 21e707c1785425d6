from .gpt import GPT, TransformerEncoder, Attention, Feedforward
from .llama import Llama, LlamaBlock
