"""Per-model parallel plans (expert parallel / tensor parallel composed with FSDP2).

Mixture-of-experts decoders, alone (``qwen3_moe``, ``qwen2_moe``, ``qwen3_5_moe`` text) or as the
language model of a multimodal wrapper (``qwen3_vl_moe``, ``qwen3_omni_moe``, ``qwen3_5_moe``,
``aero_realtime`` on a MoE backbone): experts sharded over the ``ep`` mesh (``Shard(0)`` of the
stacked parameters) and, when the data-parallel degree exceeds the expert-parallel degree,
additionally FSDP-sharded on ``dp_shard_mod_ep`` with ``Shard(1)``; attention, embeddings, the
vision / audio towers and the rest are FSDP-sharded on the full ``fsdp`` mesh.  One plan function
covers what the reference spells out per family
(src/lmms_engine/parallel/qwen3_moe/parallelize.py:26-151,
src/lmms_engine/parallel/qwen3_vl_moe/parallelize.py:34-128,
src/lmms_engine/parallel/qwen3_omni_moe/parallelize.py:1-188,
src/lmms_engine/parallel/qwen3_5_moe/parallelize.py:1-120,
src/lmms_engine/parallel/aero_realtime/parallelize.py:55-253): the decoder is found under
``language_model`` when the model is a wrapper, the towers by their attribute names.

Dense decoders (``qwen2``/``qwen3`` and the text decoder of the VL wrappers) get the
sequence-parallel tensor-parallel plan of ``parallel/tensor_parallel.py``.
"""
from __future__ import annotations

import torch

from ..utils.train_utils import str_to_dtype
from . import process_group_manager as pgm_mod
from .parallelize import register_parallel_plan


def mixed_precision_policy(args, dtype, root: bool = False):
    """FSDP2 policy of a wrapped module.  ``cast_forward_inputs`` is off: the models cast their own inputs (as they
    must under the native runtimes, which have no such hook), and FSDP's cast walks into every tensor, container and
    dataclass argument of every wrapped block - it would turn fp32 rotary tables, which the kernels read as fp32, into
    bf16 ones.  ``output_dtype`` describes what the MODEL returns, so only the root module carries it; blocks hand
    their activations on in the compute dtype."""
    from torch.distributed.fsdp import MixedPrecisionPolicy

    if dtype is None or dtype == torch.float32:
        return None
    return MixedPrecisionPolicy(param_dtype=dtype, reduce_dtype=str_to_dtype(args.reduce_dtype),
                                output_dtype=str_to_dtype(args.output_dtype) if root else None, cast_forward_inputs=False)


_mp_policy = mixed_precision_policy


def _fsdp_kwargs(args, mesh, mp):
    kw = dict(mesh=mesh, reshard_after_forward=bool((args.fsdp_config or {}).get("reshard_after_forward", True)))
    if mp is not None:
        kw["mp_policy"] = mp
    return kw


TOWER_ATTRS = ("visual", "audio_tower", "projector", "audio_projector", "multi_modal_projector")


def text_decoder(model):
    """The causal decoder of a model: the model itself, or ``language_model`` of a multimodal wrapper."""
    return getattr(model, "language_model", model)


@register_parallel_plan("qwen3_moe")
@register_parallel_plan("qwen2_moe")
@register_parallel_plan("qwen3_vl_moe")
@register_parallel_plan("qwen3_omni_moe")
@register_parallel_plan("qwen3_omni_moe_thinker")
@register_parallel_plan("qwen3_5_moe")
@register_parallel_plan("qwen3_5_moe_text")
def parallelize_moe(model, args, dtype=None, **_):
    from torch.distributed.fsdp import fully_shard
    from torch.distributed.tensor import Shard

    from ..models.moe_lm import SparseMoeBlock
    from .expert_parallel import apply_expert_parallel

    pgm = pgm_mod.process_group_manager
    if pgm.enable_tp:
        raise ValueError("tensor parallelism is not available for MoE decoders (tp_mesh must be None)")
    if pgm.enable_ep:
        apply_expert_parallel(model, pgm.ep_mesh, pgm.ep_group)
    mp = _mp_policy(args, dtype)
    fsdp_mesh = pgm.device_mesh["fsdp"]
    text = text_decoder(model)
    if text is not model:
        # towers of a multimodal wrapper: one FSDP unit each, like the reference's ``fully_shard(model.visual)``
        for attr in TOWER_ATTRS:
            tower = getattr(model, attr, None)
            if tower is not None and any(p.requires_grad for p in tower.parameters()):
                fully_shard(tower, **_fsdp_kwargs(args, fsdp_mesh, mp))
    expert_mesh = pgm.device_mesh["dp_shard_mod_ep"] if pgm.enable_ep else None
    # the token exchange hands an expert the tokens of every data-parallel rank, so its gradient is the SUM of the ranks'
    # loss gradients while every other parameter gets their mean: bring the experts to the same scale (the global norm
    # clip compares them).  The reference leaves the sum (src/lmms_engine/parallel/qwen3_moe/parallelize.py).
    dp_ranks = float(fsdp_mesh.size())
    for layer in text.model.layers:
        if isinstance(layer.mlp, SparseMoeBlock) and pgm.enable_ep:
            if expert_mesh.size() > 1:
                fully_shard(layer.mlp.experts, shard_placement_fn=lambda p: Shard(1), **_fsdp_kwargs(args, expert_mesh, mp))
                # the wrapper averages over its own mesh; the rest of the factor is applied in the experts' forward
                layer.mlp.experts.grad_scale = float(expert_mesh.size()) / dp_ranks
            else:
                # every expert lives on exactly one rank: a sharding wrapper over a mesh of one rank would only add its
                # copies, casts and gradient passes per layer (about 40 % of the step of the 30B-A3B configuration).
                # The parameters stay fp32 masters; the grouped products run in the compute dtype.
                layer.mlp.experts.compute_dtype = dtype
                layer.mlp.experts.grad_scale = 1.0 / dp_ranks
        for mixer_name in ("self_attn", "linear_attn"):  # hybrid decoders have one or the other per layer
            mixer = getattr(layer, mixer_name, None)
            if mixer is not None:
                fully_shard(mixer, **_fsdp_kwargs(args, fsdp_mesh, mp))
        if pgm.enable_ep and isinstance(layer.mlp, SparseMoeBlock):
            # the experts are managed above (or are purely expert-parallel): keep them out of the layer group
            ignored = set(layer.mlp.experts.parameters())
            fully_shard(layer, ignored_params=ignored, **_fsdp_kwargs(args, fsdp_mesh, mp))
        else:
            fully_shard(layer, **_fsdp_kwargs(args, fsdp_mesh, mp))
    if not getattr(text.config, "tie_word_embeddings", False):
        fully_shard(text.model.embed_tokens, **_fsdp_kwargs(args, fsdp_mesh, mp))
    ignored = set()
    if pgm.enable_ep:
        for m in model.modules():
            if isinstance(m, SparseMoeBlock):
                ignored |= set(m.experts.parameters())
    fully_shard(model, ignored_params=ignored or None, **_fsdp_kwargs(args, fsdp_mesh, mixed_precision_policy(args, dtype, root=True)))
    return model


@register_parallel_plan("aero_realtime")
def parallelize_aero_realtime(model, args, dtype=None, **kw):
    """Streaming-audio wrapper: expert parallelism when its backbone is a MoE decoder, the dense
    tensor-parallel plan otherwise (src/lmms_engine/parallel/aero_realtime/parallelize.py:55-253)."""
    from ..models.moe_lm import SparseMoeBlock

    if any(isinstance(m, SparseMoeBlock) for m in model.modules()):
        return parallelize_moe(model, args, dtype, **kw)
    return parallelize_dense_tp(model, args, dtype, **kw)


@register_parallel_plan("qwen2")
@register_parallel_plan("qwen3")
@register_parallel_plan("qwen3_vl")
@register_parallel_plan("qwen3_vl_text")
def parallelize_dense_tp(model, args, dtype=None, **_):
    from .tensor_parallel import apply_tensor_parallel

    return apply_tensor_parallel(model, args, dtype)
