"""Registers the stand-in modules (see ``_permissive``) before the reference is imported."""
import contextlib
import importlib.util

from . import _permissive as P


def _missing(name):
    try:
        return importlib.util.find_spec(name) is None
    except (ImportError, ValueError):
        return True


def send_to_device(obj, device, non_blocking=False, skip_keys=None):
    import torch

    if torch.is_tensor(obj):
        return obj.to(device, non_blocking=non_blocking)
    if isinstance(obj, dict):
        return type(obj)({k: send_to_device(v, device, non_blocking) for k, v in obj.items()})
    if isinstance(obj, (list, tuple)):
        return type(obj)(send_to_device(v, device, non_blocking) for v in obj)
    return obj


@contextlib.contextmanager
def init_empty_weights(include_buffers=False):
    import torch

    with torch.device("meta"):
        yield


def install_all():
    import transformers  # noqa: F401  (probe optional packages BEFORE the stand-ins exist)
    import transformers.utils.import_utils as _iu

    for fn in ("is_accelerate_available", "is_peft_available", "is_deepspeed_available"):
        try:
            getattr(_iu, fn)()
        except Exception:
            pass
    _patch_hf_device_setup()
    if _missing("hydra"):
        def main(*a, **k):
            def deco(fn):
                return fn
            return deco
        P.install("hydra", attrs={"main": main})
    if _missing("omegaconf"):
        P.install("omegaconf")
    if _missing("accelerate"):
        P.install("accelerate", submodules=("utils", "state", "accelerator", "utils.dataclasses", "utils.constants", "data_loader", "logging"),
                  attrs={"utils.send_to_device": send_to_device, "init_empty_weights": init_empty_weights})
    for name, subs in (("peft", ("tuners", "tuners.lora", "utils")), ("deepspeed", ("runtime", "runtime.zero", "runtime.zero.partition_parameters", "zero", "ops", "ops.adam")),
                       ("decord", ()), ("librosa", ()), ("soundfile", ()), ("jsonlines", ()), ("qwen_vl_utils", ("vision_process",)),
                       ("qwen_omni_utils", ()), ("av", ()), ("trl", ()), ("timm", ("models", "models.vision_transformer", "layers")), ("diffusers", ("models",)),
                       ("torchdiffeq", ()), ("bitsandbytes", ()), ("lmms_eval", ())):
        if _missing(name):
            P.install(name, submodules=subs)


def _patch_hf_device_setup():
    """``transformers.TrainingArguments`` resolves its device through accelerate's
    ``PartialState``.  Without accelerate the same answer is computed directly: the local
    CUDA device of this rank (or the CPU)."""
    import functools
    import os

    import torch
    import transformers.training_args as ta
    from transformers.utils import import_utils as iu

    if iu.is_accelerate_available():
        return

    def _setup_devices(self):
        if self.use_cpu or not torch.cuda.is_available():
            self._n_gpu = 0
            self.distributed_state = None
            return torch.device("cpu")
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        self._n_gpu = 1
        self.distributed_state = None
        return dev

    prop = functools.cached_property(_setup_devices)
    prop.__set_name__(ta.TrainingArguments, "_setup_devices")
    ta.TrainingArguments._setup_devices = prop
