"""Per-model parallel plans (expert parallel / tensor parallel composed with FSDP2).

``qwen3_moe``: experts sharded over the ``ep`` mesh (``Shard(0)`` of the stacked parameters)
and, when the data-parallel degree exceeds the expert-parallel degree, additionally
FSDP-sharded on ``dp_shard_mod_ep`` with ``Shard(1)``; attention, embeddings and the rest are
FSDP-sharded on the full ``fsdp`` mesh - the composition of the reference plan
(src/lmms_engine/parallel/qwen3_moe/parallelize.py:26-151).

Dense decoders (``qwen2``/``qwen3`` and the text decoder of the VL wrappers) get the
sequence-parallel tensor-parallel plan of ``parallel/tensor_parallel.py``.
"""
from __future__ import annotations

import torch

from ..utils.train_utils import str_to_dtype
from . import process_group_manager as pgm_mod
from .parallelize import register_parallel_plan


def _mp_policy(args, dtype):
    from torch.distributed.fsdp import MixedPrecisionPolicy

    if dtype is None or dtype == torch.float32:
        return None
    return MixedPrecisionPolicy(param_dtype=dtype, reduce_dtype=str_to_dtype(args.reduce_dtype),
                                output_dtype=str_to_dtype(args.output_dtype))


def _fsdp_kwargs(args, mesh, mp):
    kw = dict(mesh=mesh, reshard_after_forward=bool((args.fsdp_config or {}).get("reshard_after_forward", True)))
    if mp is not None:
        kw["mp_policy"] = mp
    return kw


@register_parallel_plan("qwen3_moe")
@register_parallel_plan("qwen2_moe")
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
    for layer in model.model.layers:
        if isinstance(layer.mlp, SparseMoeBlock) and pgm.enable_ep and pgm.layout.dp_shard_mod_ep > 1:
            fully_shard(layer.mlp.experts, shard_placement_fn=lambda p: Shard(1),
                        **_fsdp_kwargs(args, pgm.device_mesh["dp_shard_mod_ep"], mp))
        fully_shard(layer.self_attn, **_fsdp_kwargs(args, fsdp_mesh, mp))
        if pgm.enable_ep and isinstance(layer.mlp, SparseMoeBlock):
            # the experts are managed above (or are purely expert-parallel): keep them out of the layer group
            ignored = set(layer.mlp.experts.parameters())
            fully_shard(layer, ignored_params=ignored, **_fsdp_kwargs(args, fsdp_mesh, mp))
        else:
            fully_shard(layer, **_fsdp_kwargs(args, fsdp_mesh, mp))
    if not model.config.tie_word_embeddings:
        fully_shard(model.model.embed_tokens, **_fsdp_kwargs(args, fsdp_mesh, mp))
    ignored = set()
    if pgm.enable_ep:
        for m in model.modules():
            if isinstance(m, SparseMoeBlock):
                ignored |= set(m.experts.parameters())
    fully_shard(model, ignored_params=ignored or None, **_fsdp_kwargs(args, fsdp_mesh, mp))
    return model


@register_parallel_plan("qwen2")
@register_parallel_plan("qwen3")
@register_parallel_plan("qwen3_vl")
@register_parallel_plan("qwen3_vl_text")
def parallelize_dense_tp(model, args, dtype=None, **_):
    from .tensor_parallel import apply_tensor_parallel

    return apply_tensor_parallel(model, args, dtype)
