from . import llama     # registers "LlamaForCausalLM"
from . import tekenex   # registers "Tekenex"
from . import bevuvik   # registers "Bevuvik"
from . import fapudra   # registers "Fapudra"
