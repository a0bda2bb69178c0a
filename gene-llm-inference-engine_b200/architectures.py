"""The architectures this engine can build, entered into the one registry.

Adding an architecture means: a typed configuration class with ``from_json``, ``to_json`` and
``model_spec`` (its config.json keys translated into parts), a weight plan (its tensor names mapped
onto the parameters of those parts), and one ``register_architecture`` call like the one below.
"""
from .config import Architecture, LlamaConfig, register_architecture
from .weights.plan import llama_weight_plan

register_architecture(Architecture(
    name="LlamaForCausalLM", model_types=("llama",), config_class=LlamaConfig, weight_plan=llama_weight_plan))
