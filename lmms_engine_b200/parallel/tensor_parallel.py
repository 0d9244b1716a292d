"""Tensor-parallel plan for the dense decoders (and the text decoder of the VL wrappers).

``q/k/v/gate/up`` are column-parallel (``Shard(0)`` of the weight), ``o/down`` row-parallel
(``Shard(1)``), as in the reference plan (src/lmms_engine/parallel/qwen3_vl/parallelize.py:23-125)
with the same divisibility checks; parameters become DTensors on the ``tp`` mesh so that FSDP2
composes into 2-D shards and checkpoints record both placements.  Activations use the
sequence-parallel flavour (all-gather -> GEMM, GEMM -> reduce-scatter; see ``tp_ops``).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import process_group_manager as pgm_mod


def validate(cfg, tp: int) -> None:
    if cfg.num_attention_heads % tp or cfg.num_key_value_heads % tp:
        raise ValueError(f"attention heads ({cfg.num_attention_heads}/{cfg.num_key_value_heads}) must be divisible by tp_degree {tp}")
    if cfg.intermediate_size % tp:
        raise ValueError(f"intermediate_size ({cfg.intermediate_size}) must be divisible by tp_degree {tp}")


def shard_decoder_for_tp(decoder_lm, tp_mesh, tp_group) -> None:
    """Shard one ``DecoderLM`` in place over the tp mesh (no FSDP here)."""
    from torch.distributed.tensor import Shard, distribute_tensor

    from ..models.decoder_lm import Attention, SwiGLUMLP

    tp = tp_mesh.size()
    cfg = decoder_lm.config
    validate(cfg, tp)

    def shard(linear: nn.Linear, dim: int):
        w = nn.Parameter(distribute_tensor(linear.weight.data, tp_mesh, [Shard(dim)]), requires_grad=linear.weight.requires_grad)
        w._tp_sharded = True
        linear.weight = w
        if linear.bias is not None and dim == 0:
            b = nn.Parameter(distribute_tensor(linear.bias.data, tp_mesh, [Shard(0)]), requires_grad=linear.bias.requires_grad)
            b._tp_sharded = True
            linear.bias = b

    for m in decoder_lm.modules():
        if isinstance(m, Attention):
            for lin in (m.q_proj, m.k_proj, m.v_proj):
                shard(lin, 0)
            shard(m.o_proj, 1)
            m.n_q //= tp
            m.n_kv //= tp
        elif isinstance(m, SwiGLUMLP):
            shard(m.gate_proj, 0)
            shard(m.up_proj, 0)
            shard(m.down_proj, 1)
            m.tp_group = tp_group
    decoder_lm.tp_group = tp_group


def apply_tensor_parallel(model, args, dtype=None):
    from torch.distributed.fsdp import fully_shard

    pgm = pgm_mod.process_group_manager
    if pgm.enable_ep:
        raise ValueError("expert parallelism is not available for dense decoders")
    text = getattr(model, "language_model", model)  # VL wrappers keep the decoder here
    if pgm.enable_tp:
        shard_decoder_for_tp(text, pgm.tp_mesh, pgm.tp_group)
    from .plans import mixed_precision_policy

    mp = mixed_precision_policy(args, dtype)
    kw = dict(mesh=pgm.device_mesh["fsdp"], reshard_after_forward=bool((args.fsdp_config or {}).get("reshard_after_forward", True)))
    if mp is not None:
        kw["mp_policy"] = mp
    for layer in text.model.layers:
        fully_shard(layer, **kw)
    vis = getattr(model, "visual", None)
    if vis is not None:
        for blk in getattr(vis, "blocks", []):
            fully_shard(blk, **kw)
        fully_shard(vis, **kw)
    root_mp = mixed_precision_policy(args, dtype, root=True)
    if root_mp is not None:
        kw["mp_policy"] = root_mp
    fully_shard(model, **kw)
    return model
