"""Model registry of the engine shell (reference: models/__init__.py:1-9, core/model_runner.py:44-52)."""
from compactor_vllm.models.decoder import LlamaForCausalLM, Qwen3ForCausalLM
from compactor_vllm.models.batasun import BatasunForCausalLM
from compactor_vllm.models.fafelix import FafelixForCausalLM
from compactor_vllm.models.movolorn import MovolornForCausalLM
from compactor_vllm.models.nununex import NununexForCausalLM

MODEL_REGISTRY = {"llama": LlamaForCausalLM, "qwen3": Qwen3ForCausalLM, "movolorn": MovolornForCausalLM,
                  "batasun": BatasunForCausalLM, "fafelix": FafelixForCausalLM, "nununex": NununexForCausalLM}


def registry_key(hf_config) -> str:
    """Which entry of MODEL_REGISTRY serves a configuration (by its `model_type`)."""
    kind = str(getattr(hf_config, "model_type", "llama")).lower()
    for key in ("movolorn", "batasun", "fafelix", "nununex", "qwen3"):
        if key in kind:
            return key
    return "llama"


__all__ = ["LlamaForCausalLM", "Qwen3ForCausalLM", "MovolornForCausalLM", "BatasunForCausalLM", "FafelixForCausalLM",
           "NununexForCausalLM", "MODEL_REGISTRY",
           "registry_key"]
