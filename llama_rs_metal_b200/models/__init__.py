from . import llama  # noqa: F401  (registers LlamaForCausalLM)
from . import kikalix  # noqa: F401  (registers Kikalix)
