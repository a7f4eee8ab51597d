# SPDX-License-Identifier: Apache-2.0
"""Bi-encoder (embedding model) trainer.  Behaviour parity: projects/arctic_embed/src/arctic_embed/trainer.py:52-279,
biencoder_model_factory.py:33-77, checkpointing.py:24-39.

Every rank embeds its slice of the global batch, the embeddings are all-gathered (the local slice keeps its autograd
history), and the InfoNCE loss is taken over the *global* score matrix on every rank.  Because each rank
differentiates the global loss with respect to its own slice only, the data-parallel gradient must be the *sum* over
ranks; the engine is told so (``grad_divisor = 1``), which replaces the reference's post-backward rescaling hook.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any
from typing import Callable
from typing import Dict
from typing import List
from typing import Optional
from typing import Tuple
from typing import Union

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import Tensor

from ..checkpoint.engine import CheckpointEngine
from ..config.model import ModelConfig
from ..config.trainer import TrainerConfig
from ..logging import logger
from ..models.arch import load_arch_config
from ..models.factory import NATIVE_MODEL_TYPES
from ..models.factory import ModelFactory
from ..models.hf_io import ShardedSafetensorsWriter
from ..models.hf_io import native_to_hf
from ..models.hf_io import save_config
from ..optimizer.adam import FusedAdamOptimizerFactory
from ..scheduler.factory import HFSchedulerFactory
from ..scheduler.factory import WSDSchedulerFactory
from ..tokenizer.factory import FakeTokenizerFactory
from ..trainer.trainer import Trainer
from .data import ContrastiveLearningBatch
from .data import ContrastivePretokenizedDataConfig
from .data import ContrastivePretokenizedDataFactory
from .losses import info_nce_loss
from .losses import one_size_truncated_mrl_info_nce_loss
from .model import Biencoder
from .model import BiencoderConfig


class BiencoderModelConfig(ModelConfig):
    pooling: str = "first"
    """ ``first``, ``last`` or ``mean`` pooling of the encoder's hidden states. """


class BiencoderModelFactory(ModelFactory):
    name = "biencoder"
    config: BiencoderModelConfig

    def create_config(self):
        return load_arch_config(self.config.name_or_path, self.config.hf_config_kwargs)

    def create_model(self, model_config):
        dtype = self.config.dtype.value if hasattr(self.config.dtype, "value") else self.config.dtype
        if model_config.get("model_type") in NATIVE_MODEL_TYPES:
            from ..models.causal_lm import DecoderModel
            from ..models.hf_io import read_safetensors_dir
            from ..models.hf_io import hf_to_native_state_dict

            with torch.device(self.device):
                enc = DecoderModel(model_config, dtype=dtype)
            enc.attn_impl = self.config.attn_implementation
            if model_config.get("_source") == "preset":
                gen = torch.Generator(device=self.device).manual_seed(getattr(self.trainer.config, "seed", 42))
                with torch.no_grad():
                    for n, p in enc.named_parameters():
                        p.fill_(1.0) if "norm" in n else p.normal_(0.0, 0.02, generator=gen)
            else:
                native = hf_to_native_state_dict(read_safetensors_dir(Path(str(self.config.name_or_path))), model_config)
                own = dict(enc.named_parameters())
                with torch.no_grad():
                    for k, p in own.items():
                        src = native.get(k, native.get("model." + k))
                        if src is None:
                            raise KeyError(f"weight {k} missing from {self.config.name_or_path}")
                        p.copy_(src.to(p.dtype))
        else:
            from transformers import AutoModel

            enc = AutoModel.from_pretrained(self.config.name_or_path, dtype=dtype).to(self.device)
        model = Biencoder(enc, BiencoderConfig(pooling=self.config.pooling))
        model.activation_checkpointing = not self.config.disable_activation_checkpoint
        return model


class BiencoderCheckpointEngine(CheckpointEngine):
    """Encoder in Hugging Face layout + ``biencoder_config.json``."""

    name = "biencoder"

    @property
    def latest_checkpoint_exists(self) -> bool:
        return False

    def save(self, model) -> None:
        out = self.checkpoint_dir
        module = model.module if hasattr(model, "module") else model
        arch = module.config if isinstance(module.config, dict) else None
        writer = ShardedSafetensorsWriter(out) if self.global_rank == 0 else None
        named = model.iter_full_named_parameters() if hasattr(model, "iter_full_named_parameters") else (
            (n, p.data) for n, p in module.named_parameters())
        for name, t in named:
            if writer is None:
                continue
            name = name[len("encoder."):] if name.startswith("encoder.") else name
            for hf_name, ht in (native_to_hf(name, t, arch) if arch is not None else [(name, t)]):
                writer.add(hf_name, ht)
        if writer is not None:
            writer.finish()
            if arch is not None:
                save_config(arch, out)
            module.biencoder_config.save(out)
            logger.info(f"saved biencoder checkpoint to {out}")
        if dist.is_initialized():
            dist.barrier()

    def load(self, model: Any) -> None:
        raise NotImplementedError("biencoder checkpoints are exports; resume with the sharded engine")


class BiencoderTrainerConfig(TrainerConfig):
    type: str = "biencoder"
    use_in_batch_negatives: bool = False
    """ Treat unlabelled query/document pairs of the global batch as negatives. """
    loss_temperature: float = 0.02
    mrl_dim: Optional[int] = None
    """ Truncated dimension of the Matryoshka term (``None``: plain InfoNCE). """
    eval_interval: int = 0


def gather_embeddings(embeddings: Tensor, rank: int, world_size: int) -> Tensor:
    """All-gather ``[B_local, D]`` embeddings; the local slot keeps its autograd history."""
    embeddings = embeddings.contiguous()
    if world_size == 1:
        return embeddings
    parts = [torch.empty_like(embeddings) for _ in range(world_size)]
    dist.all_gather(parts, embeddings.detach())
    parts[rank] = embeddings
    return torch.cat(parts, dim=0)


class PeerEmbeddingGather:
    """Query and document embeddings of all ranks in ONE exchange over peer memory: every rank writes its ``q | d`` rows
    into its half of a symmetric buffer, a device-side barrier follows, and one pull kernel reads all peers' rows over
    NVLink — no library collective, no host synchronisation.  The local rows of the result keep their autograd
    history, as in :func:`gather_embeddings`."""

    def __init__(self, symm) -> None:
        from ..comm.symm import RotatingBuffers

        self.symm = symm
        self.buffers = RotatingBuffers(symm)

    def __call__(self, q: Tensor, d: Tensor, rank: int, world_size: int) -> Tuple[Tensor, Tensor]:
        nq, nd = q.numel(), d.numel()
        n = (nq + nd + 7) // 8 * 8
        buf, off = self.buffers.take("embeddings", n, q.dtype)
        mine = buf.tensor[off : off + n]
        mine[:nq].copy_(q.detach().reshape(-1))
        mine[nq : nq + nd].copy_(d.detach().reshape(-1))
        self.symm.barrier(slot=5)
        full = torch.empty(world_size * n, dtype=q.dtype, device=q.device)
        self.symm.all_gather(buf, off, n, full)
        rows = full.view(world_size, n)
        qs = [rows[r, :nq].view_as(q) for r in range(world_size)]
        ds = [rows[r, nq : nq + nd].view_as(d) for r in range(world_size)]
        qs[rank], ds[rank] = q, d
        return torch.cat(qs, dim=0), torch.cat(ds, dim=0)


def sum_gradients_cb(self: "BiencoderTrainer") -> None:
    """The loss is global on every rank: data-parallel gradients are summed, not averaged."""
    for u in self.model.units:
        u.grad_divisor = 1.0


def eval_and_log_cb(self: "BiencoderTrainer") -> None:
    every = self.config.eval_interval
    if not every or self.global_step % every != 0 or not self.eval_dataloader:
        return
    was_training = self.model.module.training
    metrics: Dict[str, float] = {}
    try:
        self.model.eval()
        for name, loader in self.eval_dataloader.items():
            vals = [self.eval(b)["infoNCE"] for b in loader]
            if vals:
                metrics[f"eval/{name}/infoNCE"] = sum(vals) / len(vals)
    finally:
        self.model.train(was_training)
    self.last_eval_metrics = metrics
    if self.wandb_experiment is not None:
        self.wandb_experiment.log(metrics, step=self.global_step)
    logger.info(f"Global Step: {self.global_step}/{self.training_horizon} Eval: {metrics}")


class BiencoderTrainer(Trainer):
    name = "biencoder"
    config: BiencoderTrainerConfig
    data_factory: ContrastivePretokenizedDataFactory
    model_factory: BiencoderModelFactory
    checkpoint_engine: BiencoderCheckpointEngine
    optimizer_factory: FusedAdamOptimizerFactory
    scheduler_factory: Union[HFSchedulerFactory, WSDSchedulerFactory]
    tokenizer_factory: FakeTokenizerFactory
    count_total_queries_seen: int = 0
    count_total_documents_seen: int = 0
    callbacks: List[Tuple[str, Callable]] = [("post-init", sum_gradients_cb), ("post-step", eval_and_log_cb)]

    def _sample_seqlens(self, batch) -> List[List[int]]:
        lens = batch.query_attention_mask.sum(1).tolist() + batch.document_attention_mask.sum(1).tolist()
        return [[int(n)] for n in lens]

    def forward_and_gather(self, batch: ContrastiveLearningBatch) -> Tuple[Tensor, Tensor, Tensor]:
        batch = batch.to_device(self.device)
        relations = batch.relevance_labels.to_dense()
        q, d = self.model(query_input_ids=batch.query_tokens, query_attention_mask=batch.query_attention_mask,
                          document_input_ids=batch.document_tokens, document_attention_mask=batch.document_attention_mask)
        symm = getattr(self.model, "symm", None)
        if symm is not None and self.world_size > 1 and q.is_cuda and q.dtype == d.dtype == torch.bfloat16:
            if getattr(self, "_peer_gather", None) is None:
                self._peer_gather = PeerEmbeddingGather(symm)
            q, d = self._peer_gather(q.contiguous(), d.contiguous(), self.global_rank, self.world_size)
        else:
            q = gather_embeddings(q, self.global_rank, self.world_size)
            d = gather_embeddings(d, self.global_rank, self.world_size)
        return q, d, relations

    @torch.no_grad()
    def eval(self, batch: ContrastiveLearningBatch) -> Dict[str, float]:
        q, d, relations = self.forward_and_gather(batch)
        scores = F.normalize(q.float(), dim=1) @ F.normalize(d.float(), dim=1).t()
        return {"infoNCE": float(info_nce_loss(scores, relations, self.config.loss_temperature))}

    def loss(self, batch: ContrastiveLearningBatch) -> Tensor:
        self.count_total_queries_seen += self.world_size * batch.query_tokens.size(0)
        self.count_total_documents_seen += self.world_size * batch.document_tokens.size(0)
        q, d, relations = self.forward_and_gather(batch)
        if self.config.use_in_batch_negatives:
            relations[relations == 0] = -1
        loss, _, _ = one_size_truncated_mrl_info_nce_loss(q, d, relations, self.config.mrl_dim,
                                                          temperature=self.config.loss_temperature)
        return loss
