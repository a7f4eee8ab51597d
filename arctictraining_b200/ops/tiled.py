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


# ---------------------------------------------------------------------------------------------------------------------
# Generic sequence-tiled autograd functions for user code: any ``fn(module, x_tile, ...)`` evaluated tile by tile.
# Call signatures follow the upstream functions the reference calls (arctic_training/model/tiled_compute.py:75-81,
# arctic_training/trainer/sft_trainer.py:145-154, projects/swiftkv/train.py:197-224).

def _seq_chunks(t: torch.Tensor, num_shards: int):
    dim = t.dim() - 2 if t.dim() >= 2 else 0
    return list(torch.chunk(t, num_shards, dim=dim)), dim


class TiledMLP(torch.autograd.Function):
    """``TiledMLP.apply(fn, module, x, num_shards, compute_params)``: ``fn(module, x)`` over ``num_shards`` tiles of
    the sequence dimension (second to last) of ``x``.  Forward keeps no intermediate activation; backward recomputes
    one tile at a time and accumulates the parameter gradients across tiles, handing each parameter its gradient
    once."""

    @staticmethod
    def forward(ctx, fn, module, x, num_shards, compute_params=None):
        ctx.fn, ctx.module, ctx.num_shards = fn, module, int(num_shards)
        ctx.params = [p for p in (compute_params or []) if p.requires_grad]
        ctx.save_for_backward(x)
        tiles, dim = _seq_chunks(x, ctx.num_shards)
        with torch.no_grad():
            outs = [fn(module, t) for t in tiles]
        return torch.cat(outs, dim=dim)

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        tiles, dim = _seq_chunks(x, ctx.num_shards)
        grads, _ = _seq_chunks(grad_out, ctx.num_shards)
        dx_parts = []
        param_grads = [None] * len(ctx.params)
        for t, g in zip(tiles, grads):
            t = t.detach().requires_grad_(True)
            with torch.enable_grad():
                y = ctx.fn(ctx.module, t)
            got = torch.autograd.grad(y, [t] + ctx.params, g, allow_unused=True)
            dx_parts.append(got[0] if got[0] is not None else torch.zeros_like(t))
            for i, pg in enumerate(got[1:]):
                if pg is not None:
                    param_grads[i] = pg if param_grads[i] is None else param_grads[i].add_(pg)
        for p, pg in zip(ctx.params, param_grads):
            if pg is not None:
                p.grad = pg if p.grad is None else p.grad.add_(pg)
        return None, None, torch.cat(dx_parts, dim=dim), None, None


class TiledFusedLogitsLoss(torch.autograd.Function):
    """``TiledFusedLogitsLoss.apply(fn, module, x, y, mask, num_shards, compute_params, output_reduction)``: a loss
    ``fn(module, x_tile, y_tile, mask_tile)`` that goes through a large projection (logits), evaluated tile by tile
    over the sequence.  The gradient of every tile is taken inside forward, so a tile's logits are freed before the
    next tile starts and ``[sequence, vocabulary]`` never exists; backward only scales the stored gradients by the
    incoming one.  ``output_reduction``: ``"sum"`` adds the tile losses, ``"mean"`` averages them weighted by tile
    length.  ``y`` is split like ``x`` when it has a sequence dimension (labels ``[B, S]`` or teacher states
    ``[B, S, H]``); ``mask`` may be ``None``; the last tile may be shorter."""

    @staticmethod
    def forward(ctx, fn, module, x, y, mask, num_shards, compute_params=None, output_reduction="mean"):
        if output_reduction not in ("sum", "mean"):
            raise ValueError(f"output_reduction must be 'sum' or 'mean', got {output_reduction!r}")
        params = [p for p in (compute_params or []) if p.requires_grad]
        num_shards = int(num_shards)
        seq_dim = x.dim() - 2
        seq_len = x.shape[seq_dim]

        def split_like_x(t):
            if t is None:
                return [None] * num_shards
            dim = next((d for d in range(t.dim()) if t.shape[d] == seq_len and d >= seq_dim - (x.dim() - t.dim())
                        and d <= seq_dim), None)
            if dim is None:
                raise ValueError(f"cannot find the sequence dimension ({seq_len}) in a tensor of shape {tuple(t.shape)}")
            return list(torch.chunk(t, num_shards, dim=dim))

        x_tiles = list(torch.chunk(x, num_shards, dim=seq_dim))
        y_tiles, m_tiles = split_like_x(y), split_like_x(mask)
        need_dx = x.requires_grad
        dx_parts = []
        param_grads = [None] * len(params)
        total = None
        for xt, yt, mt in zip(x_tiles, y_tiles, m_tiles):
            xt = xt.detach().requires_grad_(need_dx)
            with torch.enable_grad():
                loss = fn(module, xt, yt, mt)
                if output_reduction == "mean":
                    loss = loss * (xt.shape[seq_dim] / seq_len)
            wanted = ([xt] if need_dx else []) + params
            if wanted and loss.requires_grad:
                got = list(torch.autograd.grad(loss, wanted, allow_unused=True))
                if need_dx:
                    g = got.pop(0)
                    dx_parts.append(g if g is not None else torch.zeros_like(xt))
                for i, pg in enumerate(got):
                    if pg is not None:
                        param_grads[i] = pg if param_grads[i] is None else param_grads[i].add_(pg)
            elif need_dx:
                dx_parts.append(torch.zeros_like(xt))
            total = loss.detach() if total is None else total + loss.detach()
        ctx.seq_dim, ctx.params, ctx.need_dx = seq_dim, params, need_dx
        ctx.dx = torch.cat(dx_parts, dim=seq_dim) if need_dx else None
        ctx.param_grads = param_grads
        return total

    @staticmethod
    def backward(ctx, grad_out):
        for p, pg in zip(ctx.params, ctx.param_grads):
            if pg is not None:
                pg = pg * grad_out.to(pg.dtype)
                p.grad = pg if p.grad is None else p.grad.add_(pg)
        dx = ctx.dx * grad_out.to(ctx.dx.dtype) if ctx.need_dx else None
        ctx.dx, ctx.param_grads = None, []
        return None, None, dx, None, None, None, None, None
