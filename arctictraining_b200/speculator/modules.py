# SPDX-License-Identifier: Apache-2.0
"""Speculative-decoding draft heads trained on top of a frozen base model.

Two families (behaviour parity: projects/mlp_speculator/mlp_speculator/speculator.py:29-300 and
projects/arctic_lstm_speculator/speculator/speculator.py:95-348):

* ``MLPSpeculator`` / ``sum_rnn``: per head, the state is projected, the embedding of the previous ground-truth
  token is added with a fixed weight, followed by a parameterised layer norm and GELU; a vocabulary head reads the
  new state.
* ``sum_lstm``: the same recurrence with forget / input / cell / output gates (Arctic LSTM speculator).

``forward`` returns the stacked logits ``[heads, B, N, V]`` like the reference.  ``head_states`` returns the hidden
state of every head instead, so a trainer can feed them to the tiled fused linear-cross-entropy op and never build
the ``heads x tokens x vocab`` logits.
"""

from __future__ import annotations

import json
import math
import os
from typing import List
from typing import Union

import torch
import torch.nn as nn


def _dims(v: Union[int, str]) -> List[int]:
    return [v] if isinstance(v, int) else [int(x) for x in str(v).split(".")]


class LayerNormParameterized(nn.Module):
    """RMS-style normalisation with optional mean removal, scale and shift."""

    def __init__(self, normalized_shape: int, eps: float = 1e-6, elementwise_scale: bool = True,
                 elementwise_shift: bool = False, use_mean: bool = False, use_high_precision_pow: bool = False) -> None:
        super().__init__()
        self.eps, self.use_mean, self.use_high_precision_pow = eps, use_mean, use_high_precision_pow
        self.elementwise_scale, self.elementwise_shift = elementwise_scale, elementwise_shift
        if elementwise_scale:
            self.weight = nn.Parameter(torch.ones(normalized_shape))
        if elementwise_shift:
            self.bias = nn.Parameter(torch.zeros(normalized_shape))

    def reset_parameters(self) -> None:
        if self.elementwise_scale:
            self.weight.data.fill_(1)
        if self.elementwise_shift:
            self.bias.data.zero_()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.use_mean:
            x = x - x.mean(-1, keepdim=True)
        xf = x.float() if self.use_high_precision_pow else x
        x = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x)
        if self.elementwise_scale:
            x = self.weight * x
        if self.elementwise_shift:
            x = x + self.bias
        return x


class SpeculatorConfig:
    """Serialisable description of a speculator (written as ``config.json`` next to ``pytorch_model.bin``)."""

    def __init__(self, base_model_name_or_path: str, input_hidden_dim: int, inner_dim: Union[int, str],
                 proj_dim: Union[int, str], emb_dim: Union[int, str], vocab_size: int, n_predict: int,
                 tie_weights: bool = False, scale_input: bool = False, method: str = "sum_rnn",
                 tie_lstm_embs: bool = False, architecture: str = "ArcticLSTMSpeculatorPreTrainedModel") -> None:
        self.architectures = [architecture]
        self.base_model_name_or_path = str(base_model_name_or_path)
        self.input_hidden_dim = input_hidden_dim
        self.inner_dim, self.proj_dim, self.emb_dim = str(inner_dim), str(proj_dim), str(emb_dim)
        self.model_type = "mlp_speculator"
        self.n_candidates = self.n_predict = n_predict
        self.scale_input, self.tie_weights, self.tie_lstm_embs = scale_input, tie_weights, tie_lstm_embs
        self.top_k_tokens_per_head = [1] * n_predict
        self.torch_dtype = "bfloat16"
        self.vocab_size = vocab_size
        self.method = method

    def save(self, output_dir: str) -> None:
        with open(os.path.join(output_dir, "config.json"), "w") as fh:
            json.dump(self.__dict__, fh)


class Speculator(nn.Module):
    def __init__(self, config: SpeculatorConfig) -> None:
        super().__init__()
        c = self.config = config
        self.n_predict, self.input_hidden_dim = c.n_predict, c.input_hidden_dim
        self.inner_dim, self.emb_dim, self.proj_dim = _dims(c.inner_dim), _dims(c.emb_dim), _dims(c.proj_dim)
        self.vocab_size, self.scale_input = c.vocab_size, c.scale_input
        self.tie_weights, self.tie_lstm_embs, self.method = c.tie_weights, c.tie_lstm_embs, c.method
        self.activation = nn.GELU()
        H, I, P, E, V = self.input_hidden_dim, self.inner_dim[-1], self.proj_dim[0], self.emb_dim[0], self.vocab_size

        def ln(dim: int) -> LayerNormParameterized:
            return LayerNormParameterized(dim, elementwise_shift=True, elementwise_scale=True)

        def stack(dims: List[int], first: nn.Module) -> nn.Sequential:
            mods: List[nn.Module] = [first]
            for i in range(1, len(dims)):
                mods += [ln(dims[i]), self.activation, nn.Linear(dims[i - 1], dims[i], bias=False)]
            return nn.Sequential(*mods)

        n_own = 1 if self.tie_weights else self.n_predict
        n_proj = min(2, self.n_predict) if self.tie_weights else self.n_predict
        if self.method == "sum_rnn":
            self.emb = nn.ModuleList([stack(self.emb_dim, nn.Embedding(V, E)) for _ in range(n_own)])
            self.proj = nn.ModuleList(
                [stack(self.proj_dim, nn.Linear(H if i == 0 else I, P, bias=False)) for i in range(n_proj)]
            )
            self.ln = nn.ModuleList([nn.Sequential(ln(self.inner_dim[0])) for _ in range(n_own)])
        elif self.method == "sum_lstm":
            assert self.tie_weights, "sum_lstm shares its weights across heads"
            self.forget_emb = nn.ModuleList([nn.Embedding(V, E)])
            if self.tie_lstm_embs:
                self.input_emb = self.cell_emb = self.output_emb = self.forget_emb
            else:
                self.input_emb = nn.ModuleList([nn.Embedding(V, E)])
                self.cell_emb = nn.ModuleList([nn.Embedding(V, E)])
                self.output_emb = nn.ModuleList([nn.Embedding(V, E)])
            for gate in ("forget", "input", "cell", "output"):
                setattr(self, f"{gate}_proj", nn.ModuleList([nn.Linear(H, P, bias=False), nn.Linear(I, P, bias=False)]))
            self.cell_ln = nn.ModuleList([ln(self.inner_dim[0])])
            self.state_ln = nn.ModuleList([ln(self.inner_dim[0])])
        else:
            raise ValueError(f"unknown speculator method {self.method!r}")
        if self.scale_input:
            self.ln0 = LayerNormParameterized(H, elementwise_shift=False, elementwise_scale=False)
        self.head = nn.ModuleList([nn.Linear(I, V, bias=False) for _ in range(self.n_predict)])
        self.state_weight = 0.5 ** (0.5 / self.n_predict)
        self.emb_weight = math.sqrt((1 - self.state_weight**2) * (self.emb_dim[-1] / 2))
        if self.tie_weights and self.n_predict > 1:
            for h in self.head:
                h.weight = self.head[0].weight

    def reset_parameters(self) -> None:
        for m in self.modules():
            if isinstance(m, (nn.Embedding, nn.Linear)):
                nn.init.normal_(m.weight, 0, 1 / math.sqrt(min(m.weight.shape)))
            elif isinstance(m, LayerNormParameterized):
                m.reset_parameters()

    def head_states(self, state: torch.Tensor, inds: torch.Tensor) -> List[torch.Tensor]:
        """``state [B, N, H]`` from the base model, ``inds [B, N + n_predict]`` ground-truth tokens;
        returns the state each head predicts from (``n_predict`` tensors ``[B, N, inner]``)."""
        out: List[torch.Tensor] = []
        if self.scale_input:
            state = self.ln0(state) / (2**0.5)
        N = state.size(1)
        alpha = self.emb_weight / self.state_weight
        if self.method == "sum_lstm":
            cell = torch.zeros(*state.shape[:-1], self.inner_dim[-1], device=state.device, dtype=state.dtype)
            for i in range(self.n_predict):
                prev = state
                pi = 1 if i >= 1 else 0
                tok = inds[:, i : i + N]
                f = torch.sigmoid(torch.add(self.forget_proj[pi](prev), self.forget_emb[0](tok), alpha=alpha))
                g = torch.sigmoid(torch.add(self.input_proj[pi](prev), self.input_emb[0](tok), alpha=alpha))
                cand = torch.add(self.cell_proj[pi](prev), self.cell_emb[0](tok), alpha=alpha)
                cand = self.activation(self.cell_ln[0](cand)) * g
                o = torch.sigmoid(torch.add(self.output_proj[pi](prev), self.output_emb[0](tok), alpha=alpha))
                cell = cell * f + cand
                state = self.activation(self.state_ln[0](cell)) * o
                out.append(state)
            return out
        for i in range(self.n_predict):
            ei = 0 if self.tie_weights else i
            pi = min(i, 1) if self.tie_weights else i
            z = self.emb[ei](inds[:, i : i + N])
            state = torch.add(self.proj[pi](state), z, alpha=alpha)
            state = self.activation(self.ln[ei](state))
            out.append(state)
        return out

    def forward(self, state: torch.Tensor, inds: torch.Tensor) -> torch.Tensor:
        return torch.stack([self.head[i](s) for i, s in enumerate(self.head_states(state, inds))], dim=0)

    @torch.no_grad()
    def generate_suffixes(self, state: torch.Tensor, last_token: torch.Tensor) -> torch.Tensor:
        """Greedy draft of ``n_predict`` tokens from one base-model state ``[B, H]`` and the last token ``[B]``."""
        if self.method != "sum_rnn":
            raise NotImplementedError("greedy drafting is implemented for the sum_rnn family")
        if self.scale_input:
            state = self.ln0(state) / (2**0.5)
        alpha = self.emb_weight / self.state_weight
        toks = []
        tok = last_token
        for i in range(self.n_predict):
            ei = 0 if self.tie_weights else i
            pi = min(i, 1) if self.tie_weights else i
            state = self.activation(self.ln[ei](torch.add(self.proj[pi](state), self.emb[ei](tok), alpha=alpha)))
            tok = self.head[i](state).argmax(-1)
            toks.append(tok)
        return torch.stack(toks, dim=1)


class MLPSpeculatorConfig(SpeculatorConfig):
    def __init__(self, base_model_name_or_path: str, emb_dim: int, inner_dim: int, vocab_size: int, n_predict: int,
                 tie_weights: bool = False, scale_input: bool = False) -> None:
        inner = inner_dim or emb_dim
        super().__init__(base_model_name_or_path, emb_dim, inner, inner, inner, vocab_size, n_predict, tie_weights,
                         scale_input, "sum_rnn", architecture="MLPSpeculatorPreTrainedModel")


MLPSpeculator = Speculator
ArcticLSTMSpeculator = Speculator
ArcticLSTMSpeculatorConfig = SpeculatorConfig
