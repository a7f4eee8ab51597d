# SPDX-License-Identifier: Apache-2.0
"""Hugging Face export checkpoints (recipe name ``huggingface``).

Writes ``output_dir/global_step_<N>/{config.json, model.safetensors | model-0000i-of-0000N.safetensors +
model.safetensors.index.json, tokenizer files}``.  Parity: arctic_training/checkpoint/hf_engine.py:28-161.
Under ZeRO-3 the parameters are gathered one unit (decoder layer) at a time — every rank takes part in the
gathers, rank 0 streams tensors into shards of bounded size — so the full model is never resident on one
GPU.  Under expert parallelism the expert stacks of all expert-parallel ranks are gathered into the Hugging Face
per-expert names.  With PEFT only trainable tensors are written.  Loading is not supported (resume uses the sharded
engine), as in the reference.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any
from typing import Optional

import torch

from ..logging import logger
from ..models.hf_io import ShardedSafetensorsWriter
from ..models.hf_io import native_to_hf
from ..models.hf_io import save_config
from .engine import CheckpointEngine


class HFCheckpointEngine(CheckpointEngine):
    name = "huggingface"
    max_shard_bytes = 4 << 30

    @property
    def latest_checkpoint_exists(self) -> bool:
        return False

    def model_file(self, file_name: Optional[str] = None) -> Path:
        """Path of a file inside the current step's export directory (``model.pt`` when no name is given)."""
        return self.checkpoint_dir / (file_name or "model.pt")

    @property
    def config_file(self) -> Path:
        return self.checkpoint_dir / "config.json"

    @property
    def generation_config_file(self) -> Path:
        return self.checkpoint_dir / "generation_config.json"

    def _export_filter(self, model_module: torch.nn.Module):
        if getattr(self.trainer.config.model, "peft_config", None):
            trainable = {n for n, p in model_module.named_parameters() if p.requires_grad}
            return lambda name: name in trainable
        return lambda name: True

    def save(self, model) -> None:
        out_dir = self.checkpoint_dir
        module = model.module if hasattr(model, "module") else model
        cfg = getattr(module, "config", None)
        is_main = self.global_rank == 0
        keep = self._export_filter(module)
        if getattr(self.trainer.config.model, "peft_config", None):
            return self._save_adapter(model, module, out_dir, is_main)
        writer = ShardedSafetensorsWriter(out_dir, self.max_shard_bytes) if is_main else None
        arch = cfg if isinstance(cfg, dict) else None
        from ..moe.convert import expert_parallel_of
        from ..moe.convert import gather_expert_tensor

        ep_size, ep_group = expert_parallel_of(module)
        if hasattr(model, "iter_full_named_parameters"):
            named = model.iter_full_named_parameters()
        else:
            named = ((n, p.data) for n, p in module.named_parameters())
        for name, tensor in named:
            if ep_size > 1 and name.endswith(("mlp.expert_gate_up", "mlp.expert_down")):
                # every expert-parallel rank holds a slice of the expert stack: all ranks of the group join the
                # gather, the writing rank receives the experts in global order
                tensor = gather_expert_tensor(tensor, ep_size, ep_group, keep=is_main)
            if not keep(name) or writer is None:
                continue
            items = native_to_hf(name, tensor, arch) if arch is not None else [(name, tensor)]
            for hf_name, t in items:
                writer.add(hf_name, t)
        if is_main:
            writer.finish()
            if arch is not None:
                save_config(arch, out_dir, dtype=next(module.parameters()).dtype)
            elif cfg is not None and hasattr(cfg, "save_pretrained"):
                cfg.save_pretrained(out_dir)
            tok = getattr(self.trainer, "tokenizer", None)
            if tok is not None and hasattr(tok, "save_pretrained"):
                tok.save_pretrained(out_dir)
            logger.info(f"saved Hugging Face checkpoint to {out_dir}")
        from ..comm import dist as cdist

        cdist.barrier()

    def _save_adapter(self, model, module, out_dir, is_main: bool) -> None:
        """PEFT runs export the adapter only, in the layout of the ``peft`` package (``adapter_model.safetensors`` +
        ``adapter_config.json``), as the reference does through ``save_pretrained(state_dict=trainable)``."""
        from ..models.peft import save_adapter

        if hasattr(model, "iter_full_named_parameters"):
            named = model.iter_full_named_parameters()  # every rank takes part in the gathers
        else:
            named = ((n, p.data) for n, p in module.named_parameters())
        if type(module).__module__.split(".")[0] == "peft" and hasattr(module, "save_pretrained"):
            # a transformers model wrapped by the peft package: that package writes its own layout, from the gathered
            # trainable tensors (under ZeRO-3 the module's own state dict holds released, empty parameters)
            trainable = {n for n, p in module.named_parameters() if p.requires_grad}
            gathered = {n: t.detach().to("cpu").clone() for n, t in named if n in trainable}
            if is_main:
                module.save_pretrained(str(out_dir), state_dict=gathered, safe_serialization=True)
                tok = getattr(self.trainer, "tokenizer", None)
                if tok is not None and hasattr(tok, "save_pretrained"):
                    tok.save_pretrained(out_dir)
                logger.info(f"saved {len(gathered)} adapter tensors to {out_dir}")
            from ..comm import dist as cdist

            cdist.barrier()
            return
        pairs = [(n, t.detach().to("cpu").clone()) for n, t in named if ".lora_A." in n or ".lora_B." in n]
        if is_main:
            n = save_adapter(out_dir, pairs, module, str(self.trainer.config.model.name_or_path))
            tok = getattr(self.trainer, "tokenizer", None)
            if tok is not None and hasattr(tok, "save_pretrained"):
                tok.save_pretrained(out_dir)
            logger.info(f"saved {n} adapter tensors to {out_dir}")
        from ..comm import dist as cdist

        cdist.barrier()

    def load(self, model: Any) -> None:
        raise NotImplementedError("the Hugging Face engine exports only; resume with the sharded engine")
