from . import llama          # registers "LlamaForCausalLM"
from . import deganex        # registers "Deganex"
from . import lotirax        # registers "Lotirax"
from . import tubazen        # registers "Tubazen"
from . import lugizen        # registers "Lugizen"
from .text_model import TextModel
