# SPDX-License-Identifier: Apache-2.0
"""Sequence-tiled MLP: run a feed-forward block over tiles of the sequence so that the
``[tokens, intermediate]`` activations exist for one tile at a time; the backward pass recomputes each tile.

Behaviour parity: arctic_training/model/tiled_compute.py:27-102 (tile count ``ceil(seqlen / hidden)``).
The tile count is a pure function of shapes, so all ranks agree without the per-layer all-reduce the
reference needs to keep ZeRO-3 ranks in lock-step.
"""

from __future__ import annotations

import math
import types

import torch
import torch.nn as nn


class _TiledMLPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mlp: nn.Module, x: torch.Tensor, num_tiles: int, *params: torch.Tensor):
        ctx.mlp, ctx.num_tiles = mlp, num_tiles
        ctx.save_for_backward(x)
        shp = x.shape
        flat = x.reshape(-1, shp[-1])
        outs = []
        with torch.no_grad():
            for tile in torch.chunk(flat, num_tiles, dim=0):
                outs.append(mlp(tile))
        return torch.cat(outs, dim=0).view(*shp[:-1], outs[0].shape[-1])

    @staticmethod
    def backward(ctx, gout: torch.Tensor):
        (x,) = ctx.saved_tensors
        mlp, num_tiles = ctx.mlp, ctx.num_tiles
        shp = x.shape
        flat = x.reshape(-1, shp[-1])
        gflat = gout.reshape(-1, gout.shape[-1])
        dx = torch.empty_like(flat)
        params = [p for p in mlp.parameters() if p.requires_grad]
        x_tiles = torch.chunk(flat, num_tiles, dim=0)
        g_tiles = torch.chunk(gflat, num_tiles, dim=0)
        offset = 0
        for xt, gt in zip(x_tiles, g_tiles):
            xt = xt.detach().requires_grad_(True)
            with torch.enable_grad():
                yt = mlp(xt)
            # parameter gradients accumulate straight into ``p.grad`` (the engine's flat buffer)
            torch.autograd.backward(yt, gt)
            dx[offset : offset + xt.shape[0]] = xt.grad
            offset += xt.shape[0]
        return (None, dx.view(shp), None) + tuple(None for _ in params)


def num_mlp_tiles(x: torch.Tensor) -> int:
    tokens = x.numel() // x.shape[-1]
    return max(1, math.ceil(tokens / x.shape[-1]))


def tiled_mlp(mlp: nn.Module, x: torch.Tensor) -> torch.Tensor:
    tiles = num_mlp_tiles(x)
    if tiles <= 1:
        return mlp(x)
    if not torch.is_grad_enabled() or not x.requires_grad:
        flat = x.reshape(-1, x.shape[-1])
        out = torch.cat([mlp(t) for t in torch.chunk(flat, tiles, dim=0)], dim=0)
        return out.view(*x.shape[:-1], out.shape[-1])
    params = [p for p in mlp.parameters() if p.requires_grad]
    return _TiledMLPFn.apply(mlp, x, tiles, *params)


def enable_tiled_mlp_compute(model: nn.Module) -> int:
    """Patch every ``*MLP`` module of a generic (e.g. ``transformers``) model to run tiled.  Returns the
    number of modules patched."""
    count = 0
    for mod in model.modules():
        if type(mod).__name__.endswith("MLP") and not getattr(mod, "_atb_tiled", False):
            orig = mod.forward

            class _Shim(nn.Module):
                def __init__(self, owner, fwd):
                    super().__init__()
                    object.__setattr__(self, "_owner", owner)
                    self._fwd = fwd

                def parameters(self, recurse: bool = True):
                    return self._owner.parameters(recurse)

                def forward(self, t):
                    return self._fwd(t)

            shim = _Shim(mod, orig)
            mod.forward = types.MethodType(lambda self, x, _s=shim: tiled_mlp(_s, x), mod)
            mod._atb_tiled = True
            count += 1
    return count
