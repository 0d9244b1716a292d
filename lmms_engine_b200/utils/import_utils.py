"""Probes for optional packages and for this engine's own native libraries.

The reference gates code paths on external kernel packages (src/lmms_engine/utils/import_utils.py:29-86:
``is_flash_attn_2_available``, ``is_liger_kernel_available``, ...).  Here the kernels are the engine's own, so those
probes answer from the native build: attention / fused losses are "available" when the sm_100a libraries load on a
CUDA device.  The remaining probes cover packages the data plane may use."""
from __future__ import annotations

import importlib.metadata
import importlib.util
from functools import lru_cache

from packaging.version import Version


@lru_cache(maxsize=None)
def is_package_available(name: str) -> bool:
    return importlib.util.find_spec(name) is not None


def package_version(name: str) -> Version:
    try:
        return Version(importlib.metadata.version(name))
    except Exception:
        return Version("0.0.0")


@lru_cache(maxsize=None)
def is_native_available() -> bool:
    """The engine's CUDA libraries are built (or can be) and a CUDA device is present."""
    import torch

    if not torch.cuda.is_available():
        return False
    from .. import _native

    return bool(_native.have_cuda_libs())


def is_flash_attn_2_available() -> bool:
    """Varlen attention on the GPU: this engine's tcgen05 kernels."""
    return is_native_available()


def is_liger_kernel_available() -> bool:
    """Fused norms / rotary / SwiGLU / linear + cross-entropy: this engine's kernels."""
    return is_native_available()


def is_fused_moe_available() -> bool:
    """Grouped expert GEMMs: ``csrc/moe.cu``."""
    return is_native_available()


def is_torch_npu_available() -> bool:
    return False


def is_diffusers_available() -> bool:
    return is_package_available("diffusers")


def is_video_audio_available() -> bool:
    """Decoders for video and audio files (OpenCV or decord, soundfile or the standard ``wave`` module)."""
    return is_package_available("cv2") or is_package_available("decord")


def is_torch_version_greater_than(value: str) -> bool:
    return package_version("torch") > Version(value)


def is_transformers_version_greater_or_equal_to(value: str) -> bool:
    return package_version("transformers") >= Version(value)
