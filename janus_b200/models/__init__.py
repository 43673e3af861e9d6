from . import buludra, llama, mugedra, ramolix, zivitar  # noqa: F401  (registers Buludra, LlamaForCausalLM, Mugedra, Ramolix and Zivitar)
