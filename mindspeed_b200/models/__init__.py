from .gpt_model import GPTModel  # noqa: F401
from .transformer import TransformerBlock, TransformerLayer  # noqa: F401
