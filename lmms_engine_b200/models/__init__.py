"""Native model families and their registration."""
from ..mapping_func import register_model
from .config import ModelConfig
from .decoder_lm import DecoderConfig, DecoderLM

for _mt in ("qwen2", "qwen2_5", "qwen3", "llama"):
    register_model(_mt, DecoderConfig, DecoderLM, "causal_lm")

from .moe_lm import MoEConfig, MoEDecoderLM

for _mt in ("qwen3_moe", "qwen2_moe"):
    register_model(_mt, MoEConfig, MoEDecoderLM, "causal_lm")

from .vl import VLConfig, VLModel

for _mt in ("qwen2_5_vl", "qwen2_vl", "qwen3_vl", "qwen3_vl_moe", "llavaonevision1_5"):
    register_model(_mt, VLConfig, VLModel, "image_text_to_text")

from .bagel import Bagel, BagelConfig
from .diffusion import RaeAutoencoder, RaeConfig, SiT, SiTConfig, WanConfig, WanDiT
from .dllm import DiffusionLM, DLLMConfig

for _mt in ("qwen3_dllm", "dream_dllm", "llada_dllm"):
    register_model(_mt, DLLMConfig, DiffusionLM, "masked_lm")
register_model("sit", SiTConfig, SiT, "general")
from .wan import WanVideoConfig, WanVideoModel  # noqa: E402

register_model("wanvideo", WanVideoConfig, WanVideoModel, "general")
register_model("wan_dit_lite", WanConfig, WanDiT, "general")
from .rae import RaeSiglip, RaeSiglipConfig  # noqa: E402

register_model("rae_siglip", RaeSiglipConfig, RaeSiglip, "general")
register_model("rae_toy", RaeConfig, RaeAutoencoder, "general")
register_model("bagel", BagelConfig, Bagel, "general")

__all__ = ["ModelConfig", "DecoderConfig", "DecoderLM", "MoEConfig", "MoEDecoderLM", "VLConfig", "VLModel", "DLLMConfig",
           "DiffusionLM", "SiT", "SiTConfig", "WanDiT", "WanConfig", "RaeAutoencoder", "RaeConfig", "Bagel", "BagelConfig"]
from .nanovlm import Nanovlm, NanovlmConfig  # noqa: E402

register_model("nanovlm", NanovlmConfig, Nanovlm, "image_text_to_text")
from .audio import Qwen2AudioConfig, Qwen2AudioModel  # noqa: E402

register_model("qwen2_audio", Qwen2AudioConfig, Qwen2AudioModel, "general")
from .audio import AeroConfig, AeroModel  # noqa: E402

register_model("aero", AeroConfig, AeroModel, "general")
from .omni import OmniThinker, OmniThinkerConfig  # noqa: E402

for _mt in ("qwen2_5_omni_thinker", "qwen2_5_omni"):
    register_model(_mt, OmniThinkerConfig, OmniThinker, "general")
from .llava_ov import LlavaOnevision, LlavaOnevisionConfig  # noqa: E402

register_model("llava_onevision", LlavaOnevisionConfig, LlavaOnevision, "image_text_to_text")
from .omni import Omni3Thinker, Omni3ThinkerConfig  # noqa: E402

for _mt in ("qwen3_omni_moe_thinker", "qwen3_omni_moe"):
    register_model(_mt, Omni3ThinkerConfig, Omni3Thinker, "general")
from .audio import VoxtralRealtimeEncoder, VoxtralRealtimeEncoderConfig  # noqa: E402

register_model("voxtral_realtime_encoder", VoxtralRealtimeEncoderConfig, VoxtralRealtimeEncoder, "general")
from .qwen3_5 import Qwen35Config, Qwen35LM  # noqa: E402

for _mt in ("qwen3_5_text", "qwen3_5"):
    register_model(_mt, Qwen35Config, Qwen35LM, "causal_lm")
from .qwen3_5 import Qwen35MoEConfig, Qwen35MoELM  # noqa: E402

for _mt in ("qwen3_5_moe_text", "qwen3_5_moe"):
    register_model(_mt, Qwen35MoEConfig, Qwen35MoELM, "causal_lm")
for _mt in ("qwen3_5", "qwen3_5_moe"):
    register_model(_mt, VLConfig, VLModel, "image_text_to_text")

from .aero_realtime import AeroRealtimeConfig, AeroRealtimeModel  # noqa: E402

register_model("aero_realtime", AeroRealtimeConfig, AeroRealtimeModel, "image_text_to_text")

from .gated_deltanet import GatedDeltaNetConfig, GatedDeltaNetLM  # noqa: E402

register_model("gated_deltanet", GatedDeltaNetConfig, GatedDeltaNetLM, "causal_lm")

from .llava_ov2 import LlavaOnevision2  # noqa: E402

register_model("llava_onevision2", VLConfig, LlavaOnevision2, "image_text_to_text")


# ---- the class names the reference exports from its ``models`` package (src/lmms_engine/models/__init__.py) -----------------
_REFERENCE_NAMES = {
    "AeroForConditionalGeneration": ("audio", "AeroModel"), "AeroConfig": ("audio", "AeroModel.config_class"),
    "AeroProcessor": ("..datasets.extra", "Qwen2AudioProcessor"),
    "AeroRealtimeForConditionalGeneration": ("aero_realtime", "AeroRealtimeModel"),
    "AeroRealtimeProcessor": ("..datasets.realtime", "AeroRealtimeProcessor"),
    "NanovlmForConditionalGeneration": ("nanovlm", "Nanovlm"),
    "Qwen2_5OmniThinkerConfig": ("omni", "OmniThinkerConfig"), "Qwen2_5OmniThinkerForConditionalGeneration": ("omni", "OmniThinker"),
    "Qwen3OmniMoeThinkerConfig": ("omni", "Omni3ThinkerConfig"), "Qwen3OmniMoeThinkerForConditionalGeneration": ("omni", "Omni3Thinker"),
    "RaeSiglipModel": ("rae", "RaeSiglip"), "SiTModel": ("diffusion", "SiT"),
    "WanVideoForConditionalGeneration": ("wan", "WanVideoModel"),
    "WanVideoProcessor": ("..datasets.processor.generative_processors", "WanVideoProcessor"),
    "Qwen3DLLMConfig": ("dllm", "DLLMConfig"), "DreamDLLMConfig": ("dllm", "DLLMConfig"), "LLaDADLLMConfig": ("dllm", "DLLMConfig"),
    "Qwen3DLLMForMaskedLM": ("dllm", "DiffusionLM"), "DreamDLLMForMaskedLM": ("dllm", "DiffusionLM"), "LLaDADLLMForMaskedLM": ("dllm", "DiffusionLM"),
    "Llavaonevision1_5Config": ("vl", "VLConfig"), "LLaVAOneVision1_5_ForConditionalGeneration": ("vl", "VLModel"),
    "MONKEY_PATCHER": ("monkey_patch", "MONKEY_PATCHER"),
}


def __getattr__(name):
    import importlib

    if name in _REFERENCE_NAMES:
        module, attr = _REFERENCE_NAMES[name]
        package = __name__ if not module.startswith("..") else __name__.rsplit(".", 1)[0]
        obj = importlib.import_module("." + module.lstrip("."), package)
        for part in attr.split("."):
            obj = getattr(obj, part)
        return obj
    if name.startswith("apply_liger_kernel_to_"):
        from .monkey_patch import native_kernels_apply

        return native_kernels_apply(name[len("apply_liger_kernel_to_"):])
    raise AttributeError(name)
