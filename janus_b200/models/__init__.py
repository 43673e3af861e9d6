from . import llama, mugedra, ramolix, zivitar  # noqa: F401  (registers LlamaForCausalLM, Mugedra, Ramolix and Zivitar)
