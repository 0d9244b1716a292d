"""Pluecker ray embedding ``[B, V, H, W, 6] = [o x d, d]`` for camera control.

``plucker_rays`` runs the sm_100a kernel of ``csrc/camera.cu`` for CUDA inputs and the fp32
PyTorch formulation otherwise (the oracle; the reference computes it on the CPU,
src/lmms_engine/models/wanvideo/wan_video_camera_controller.py:152-184).  Helpers for relative
poses and intrinsics rescaling follow ``get_relative_pose`` / ``process_pose_file`` (:133-234).
"""
from __future__ import annotations

import numpy as np
import torch

from . import _cuda

_cuda.register("b200_plucker", "camera", "ppplii" + "is")


def plucker_rays_ref(K: torch.Tensor, c2w: torch.Tensor, H: int, W: int) -> torch.Tensor:
    B, V = K.shape[:2]
    dev, dt = c2w.device, torch.float32
    j, i = torch.meshgrid(torch.arange(H, device=dev, dtype=dt), torch.arange(W, device=dev, dtype=dt), indexing="ij")
    i = i.reshape(1, 1, H * W) + 0.5
    j = j.reshape(1, 1, H * W) + 0.5
    fx, fy, cx, cy = K.float().chunk(4, dim=-1)
    d = torch.stack(((i - cx) / fx, (j - cy) / fy, torch.ones_like(i).expand(B, V, H * W)), -1)
    d = d / d.norm(dim=-1, keepdim=True)
    rays_d = d @ c2w.float()[..., :3, :3].transpose(-1, -2)
    rays_o = c2w.float()[..., :3, 3][:, :, None].expand_as(rays_d)
    return torch.cat([torch.linalg.cross(rays_o, rays_d), rays_d], -1).reshape(B, V, H, W, 6)


def plucker_rays(K: torch.Tensor, c2w: torch.Tensor, H: int, W: int, channels_first: bool = False) -> torch.Tensor:
    """``K [B,V,4]`` = (fx, fy, cx, cy), ``c2w [B,V,4,4]``.  ``channels_first`` gives [B,V,6,H,W]."""
    B, V = K.shape[:2]
    if K.is_cuda:
        Kc, Mc = K.float().contiguous(), c2w.float().contiguous()
        shape = (B, V, 6, H, W) if channels_first else (B, V, H, W, 6)
        out = torch.empty(shape, dtype=torch.float32, device=K.device)
        _cuda.call("b200_plucker", Kc.data_ptr(), Mc.data_ptr(), out.data_ptr(), B * V, H, W, int(channels_first), _cuda.stream())
        return out
    out = plucker_rays_ref(K, c2w, H, W)
    return out.permute(0, 1, 4, 2, 3).contiguous() if channels_first else out


def relative_poses(w2c: np.ndarray) -> np.ndarray:
    """Camera-to-world matrices relative to the first camera (which becomes the identity)."""
    c2w = np.linalg.inv(w2c)
    out = [np.eye(4, dtype=np.float32)] + [w2c[0] @ m for m in c2w[1:]]
    return np.asarray(out, dtype=np.float32)


def rescale_intrinsics(fx, fy, cx, cy, orig_hw, target_hw):
    """Normalised intrinsics of a pose file -> pixel intrinsics of the target size, keeping the
    field of view of the shorter relative side."""
    oh, ow = orig_hw
    th, tw = target_hw
    if ow / oh > tw / th:  # crop width
        fx = fx * (ow / oh) / (tw / th)
    else:
        fy = fy * (tw / th) / (ow / oh)
    return fx * tw, fy * th, cx * tw, cy * th
