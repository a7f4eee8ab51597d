# SPDX-License-Identifier: Apache-2.0
"""Worker run by the multi-process CPU tests (Gloo, world size 2..4).  Usage:
``python tests/dist_worker.py <scenario> <out_dir>`` under the framework's launcher."""

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from arctictraining_b200.comm.dist import init_distributed  # noqa: E402
from arctictraining_b200.engine import TrainingEngine  # noqa: E402
from arctictraining_b200.models.arch import load_arch_config  # noqa: E402
from arctictraining_b200.models.causal_lm import CausalLM  # noqa: E402
from arctictraining_b200.optimizer.adam import FusedAdamW  # noqa: E402
from arctictraining_b200.optimizer.factory import OptimizerFactory  # noqa: E402


def make_engine(stage, gas=1, seed=0, preset="tiny-llama", **kw):
    cfg = load_arch_config(preset)
    m = CausalLM(cfg, dtype=torch.float32)
    m.init_weights(seed=seed)
    opt = FusedAdamW(OptimizerFactory.get_optimizer_grouped_params(m, 0.1), lr=1e-2, betas=(0.9, 0.95))
    return TrainingEngine(m, opt, None, {"zero_optimization": {"stage": stage}, "gradient_accumulation_steps": gas,
                                         "gradient_clipping": 1.0, **kw})


def global_batches(n, world, bs=2, seq=32, vocab=1024, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(8, vocab, (bs * world, seq), generator=g)
        labels = ids.clone()
        labels[:, : seq // 2] = -100
        out.append({"input_ids": ids, "labels": labels})
    return out


def scenario_zero(out_dir, stage, keep=0):
    rank, world = dist.get_rank(), dist.get_world_size()
    engine = make_engine(stage, activation_checkpoint_keep=keep)
    losses = []
    for b in global_batches(3, world):
        local = {k: v[rank::world] for k, v in b.items()}
        # every rank normalises by its own token count; make the counts equal so the mean of means is the global mean
        out = engine(**local)
        engine.backward(out.loss)
        engine.step()
        t = out.loss.detach().clone()
        dist.all_reduce(t)
        losses.append(float(t) / world)
    released = [u.flat is None for u in engine.units if u.name.startswith("layer")]
    params = {n: t.clone() for n, t in engine.iter_full_named_parameters()}
    if rank == 0:
        torch.save({"losses": losses, "params": params, "released": released, "norm": engine.get_global_grad_norm()},
                   Path(out_dir) / f"zero{stage}.pt")


def scenario_resume(out_dir):
    rank, world = dist.get_rank(), dist.get_world_size()
    data = [{k: v[rank::world] for k, v in b.items()} for b in global_batches(4, world)]

    def run(e, items):
        res = []
        for b in items:
            out = e(**b)
            e.backward(out.loss)
            e.step()
            res.append(float(out.loss))
        return res

    a = make_engine(3)
    run(a, data[:2])
    a.save_checkpoint(Path(out_dir) / "ckpt", tag="t", client_state={"k": 1})
    rest_a = run(a, data[2:])
    b = make_engine(3, seed=99)
    _, cs = b.load_checkpoint(Path(out_dir) / "ckpt")
    rest_b = run(b, data[2:])
    ok = rest_a == rest_b and cs == {"k": 1}
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        (Path(out_dir) / "resume.json").write_text(json.dumps({"ok": all(flags), "a": rest_a, "b": rest_b}))


def scenario_trainer(out_dir, recipe_path):
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    cfg = get_config(Path(recipe_path))
    trainer = get_registered_trainer(cfg.type)(cfg)
    trainer.train()


def scenario_rank_failure(out_dir):
    """Rank 1 raises before the first collective of the step; the launcher must take the job down."""
    if dist.get_rank() == 1:
        raise RuntimeError("injected failure on rank 1")
    import time

    time.sleep(60)


def scenario_ulysses_hf(out_dir):
    """A model of the transformers library under sequence parallelism: every rank holds a slice of a packed sequence;
    loss and summed gradients must match the same model run on the whole sequence in one process."""
    from transformers import LlamaConfig
    from transformers import LlamaForCausalLM

    from arctictraining_b200.parallel.ulysses import UlyssesContext
    from arctictraining_b200.parallel.ulysses import shard_batch_for_rank
    from arctictraining_b200.parallel.ulysses_hf import chunked_causal_lm_loss_sum
    from arctictraining_b200.parallel.ulysses_hf import enable_ulysses_for_hf_model

    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = LlamaConfig(vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=1, max_position_embeddings=128, attn_implementation="sdpa")
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg)
    S = 48
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 160, (1, S), generator=g)
    position_ids = torch.cat([torch.arange(20), torch.arange(S - 20)])[None]  # two packed samples
    labels = ids.clone()
    labels[0, :4] = -100
    labels[0, 20] = -100  # the first token of a sample is no target of the sample before it
    batch = {"input_ids": ids, "position_ids": position_ids, "labels": labels}

    # in this process: the two packed samples run one by one, so neither can attend to the other (the library's own
    # attention functions do not all isolate packed samples; the registered function must)
    logits = torch.cat([model(input_ids=ids[:, :20]).logits, model(input_ids=ids[:, 20:]).logits], dim=1).float()
    shift = torch.nn.functional.pad(labels[:, 1:], (0, 1), value=-100)
    shift[0, 19] = -100
    ref_sum = torch.nn.functional.cross_entropy(logits[0], shift[0], ignore_index=-100, reduction="sum")
    ref_loss = ref_sum / (shift != -100).sum()
    ref_loss.backward()
    ref_grads = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()

    ctx = UlyssesContext(dist.group.WORLD, world, rank)
    fn = enable_ulysses_for_hf_model(model, ctx, "sdpa")
    local = shard_batch_for_rank(dict(batch), rank, world)
    sl = shift[:, rank * (S // world):(rank + 1) * (S // world)]
    hidden = model.model(input_ids=local["input_ids"], position_ids=local["position_ids"], use_cache=False).last_hidden_state
    loss_sum, n = chunked_causal_lm_loss_sum(model.lm_head, hidden, sl, logits_bytes_per_chunk=4 * 160 * 7)
    loss = ctx.aggregate_loss(loss_sum, n)
    loss.backward()
    grads = {}
    for name, p in model.named_parameters():
        gsum = p.grad.clone()
        dist.all_reduce(gsum)
        grads[name] = gsum
    # the call shape of the upstream helper: registered by name before the model exists, the function takes the place
    # of the core implementation, so a model created with that implementation afterwards attends through it
    from arctictraining_b200.parallel.ulysses_hf import UlyssesSPAttentionHF

    mpu = UlyssesSPAttentionHF.register_with_transformers("some/model", "sdpa", world, 1, S)
    assert mpu.get_sequence_parallel_world_size() == world and mpu.get_sequence_parallel_rank() == rank
    cfg2 = LlamaConfig(vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=1, max_position_embeddings=128, attn_implementation="sdpa")
    torch.manual_seed(0)
    model2 = LlamaForCausalLM(cfg2)
    assert model2.config._attn_implementation == "sdpa"
    with torch.no_grad():
        hidden2 = model2.model(input_ids=local["input_ids"], position_ids=local["position_ids"], use_cache=False).last_hidden_state
    same = bool(torch.allclose(hidden2, hidden.detach(), rtol=1e-5, atol=1e-6)) and mpu.attention.calls >= 2
    flag = torch.tensor([1.0 if same else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"ref_loss": ref_loss.detach(), "loss": loss.detach(), "ref_grads": ref_grads, "grads": grads,
                    "calls": fn.calls, "registered_by_name_matches": bool(flag.item())}, Path(out_dir) / "ulysses_hf.pt")


def scenario_shim(out_dir):
    """User code written against the upstream engine package: its imports resolve to the stand-in modules.  Rank 0
    overwrites a stage-3 parameter inside ``GatheredParameters(modifier_rank=0)``; every rank then sees the new value,
    also after a training step (the master weights were refreshed)."""
    from arctictraining_b200.compat import deepspeed_shim

    assert deepspeed_shim.install()
    import deepspeed.comm as ds_dist
    from deepspeed.accelerator import get_accelerator
    from deepspeed.runtime.zero import GatheredParameters

    rank = ds_dist.get_rank()
    assert get_accelerator().communication_backend_name() == "gloo"
    engine = make_engine(3)
    layer = engine.module.model.layers[1]
    target = layer.mlp.down_proj.weight if hasattr(layer.mlp, "down_proj") else next(layer.parameters())
    name = next(n for n, p in engine.module.named_parameters() if p is target)
    assert target.numel() == 0  # released between steps under stage 3
    with GatheredParameters([target], modifier_rank=0):
        assert target.numel() > 0
        if rank == 0:
            target.data.fill_(0.125)
    assert target.numel() == 0
    seen = dict(engine.iter_full_named_parameters())[name].clone()
    with GatheredParameters([target]):  # read-only access
        inside = target.detach().clone()
    b = global_batches(1, ds_dist.get_world_size())[0]
    out = engine(**{k: v[rank::ds_dist.get_world_size()] for k, v in b.items()})
    engine.backward(out.loss)
    engine.step()
    after = dict(engine.iter_full_named_parameters())[name].clone()
    torch.save({"seen": seen, "inside": inside, "after": after}, Path(out_dir) / f"shim_rank{rank}.pt")


def main():
    scenario, out_dir = sys.argv[1], sys.argv[2]
    init_distributed(timeout_s=60)
    if scenario == "zero3keep":
        scenario_zero(out_dir, 3, keep=2)  # writes zero3.pt
    elif scenario.startswith("zero"):
        scenario_zero(out_dir, int(scenario[4:]))
    elif scenario == "resume":
        scenario_resume(out_dir)
    elif scenario == "trainer":
        scenario_trainer(out_dir, sys.argv[3])
    elif scenario == "rank_failure":
        scenario_rank_failure(out_dir)
    elif scenario == "shim":
        scenario_shim(out_dir)
    elif scenario == "ulysses_hf":
        scenario_ulysses_hf(out_dir)
    else:
        raise SystemExit(f"unknown scenario {scenario}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    # the launcher appends --local_rank=N
    sys.argv = [a for a in sys.argv if not a.startswith("--local_rank")]
    main()
