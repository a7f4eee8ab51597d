# SPDX-License-Identifier: Apache-2.0
"""Engine correctness on CPU: the flat-buffer engine must reproduce plain PyTorch training, and the ZeRO
stages / checkpointing / accumulation variants must agree with each other."""

import copy

import pytest
import torch

from arctictraining_b200.engine import TrainingEngine
from arctictraining_b200.models.arch import load_arch_config
from arctictraining_b200.models.causal_lm import CausalLM
from arctictraining_b200.optimizer.adam import FusedAdamW
from arctictraining_b200.optimizer.factory import OptimizerFactory


def make_model(seed=0, **overrides):
    cfg = load_arch_config("tiny-llama", overrides)
    m = CausalLM(cfg, dtype=torch.float32)
    m.init_weights(seed=seed)
    return m


def make_engine(model, stage, gas=1, clip=1.0, ckpt=True, lr=1e-2, wd=0.1, tiled=False, keep=0):
    model.activation_checkpointing = ckpt
    model.tiled_mlp = tiled
    groups = OptimizerFactory.get_optimizer_grouped_params(model, wd)
    opt = FusedAdamW(groups, lr=lr, betas=(0.9, 0.95))
    return TrainingEngine(model, opt, None, {
        "zero_optimization": {"stage": stage}, "gradient_accumulation_steps": gas, "gradient_clipping": clip,
        "activation_checkpoint_keep": keep,
    })


def batches(n, bs=2, seq=32, vocab=1024, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(8, vocab, (bs, seq), generator=g)
        labels = ids.clone()
        labels[:, : seq // 2] = -100
        out.append({"input_ids": ids, "labels": labels})
    return out


def run(engine, data):
    losses = []
    for b in data:
        out = engine(**b)
        engine.backward(out.loss)
        engine.step()
        losses.append(float(out.loss))
    return losses


def full_params(engine):
    return {n: t.clone() for n, t in engine.iter_full_named_parameters()}


def test_engine_matches_plain_pytorch():
    data = batches(4)
    ref = make_model()
    eng_model = copy.deepcopy(ref)
    groups = OptimizerFactory.get_optimizer_grouped_params(ref, 0.1)
    opt = torch.optim.AdamW(groups, lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    ref_losses = []
    for b in data:
        out = ref(**b)
        opt.zero_grad()
        out.loss.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
        ref_losses.append(float(out.loss))
    engine = make_engine(eng_model, stage=0)
    losses = run(engine, data)
    assert losses == pytest.approx(ref_losses, rel=1e-4, abs=1e-5)
    mine = full_params(engine)
    for n, p in ref.named_parameters():
        assert torch.allclose(mine[n], p.data, atol=2e-5, rtol=1e-4), n


@pytest.mark.parametrize("stage", [1, 2, 3])
def test_zero_stages_agree_with_stage0(stage):
    data = batches(3)
    base = run(make_engine(make_model(), 0), data)
    assert run(make_engine(make_model(), stage), data) == pytest.approx(base, rel=1e-5)


def test_checkpointing_and_tiled_mlp_do_not_change_results():
    data = batches(3, seq=160)
    a = make_engine(make_model(), 3, ckpt=True)
    b = make_engine(make_model(), 0, ckpt=False)
    c = make_engine(make_model(), 3, ckpt=True, tiled=True)
    la, lb, lc = run(a, data), run(b, data), run(c, data)
    assert la == pytest.approx(lb, rel=1e-5)
    assert lc == pytest.approx(lb, rel=1e-5)
    pa, pb, pc = full_params(a), full_params(b), full_params(c)
    for n in pa:
        assert (pa[n] - pb[n]).abs().mean() < 1e-5, n
        # tiling changes the summation order of weight gradients; Adam turns that into small parameter noise
        assert (pc[n] - pb[n]).abs().mean() < 1e-4, n


@pytest.mark.parametrize("keep", [1, 2, 100])
def test_keeping_activations_of_some_layers_does_not_change_results(keep):
    data = batches(3)
    a = make_engine(make_model(), 3, ckpt=True, keep=0)
    b = make_engine(make_model(), 3, ckpt=True, keep=keep, gas=1)
    assert run(b, data) == pytest.approx(run(a, data), rel=1e-6)
    pa, pb = full_params(a), full_params(b)
    for n in pa:
        assert (pa[n] - pb[n]).abs().max() < 1e-6, n


def test_gradient_accumulation_equals_big_batch():
    data = batches(4, bs=2)
    big = [{k: torch.cat([data[i][k], data[i + 1][k]]) for k in data[0]} for i in (0, 2)]
    e_big = make_engine(make_model(), 0, gas=1)
    e_acc = make_engine(make_model(), 2, gas=2)
    run(e_big, big)
    run(e_acc, data)
    assert e_acc.global_steps == 2 and e_big.global_steps == 2
    pb, pa = full_params(e_big), full_params(e_acc)
    for n in pb:
        assert torch.allclose(pa[n], pb[n], atol=5e-5, rtol=1e-3), n


def test_grad_norm_is_reported_and_clipping_applies():
    data = batches(1)
    e = make_engine(make_model(), 0, clip=1e-3, lr=1.0, wd=0.0)
    before = full_params(e)
    run(e, data)
    assert e.get_global_grad_norm() > 1e-3
    after = full_params(e)
    # with Adam the first update has magnitude ~lr regardless of the clip, so only check it ran and is finite
    assert all(torch.isfinite(after[n]).all() for n in after)
    assert any(not torch.equal(after[n], before[n]) for n in after)


def test_frozen_parameters_get_no_state_and_do_not_move():
    m = make_model()
    for p in m.model.embed_tokens.parameters():
        p.requires_grad_(False)
    e = make_engine(m, 2)
    emb_before = m.model.embed_tokens.weight.detach().clone()
    run(e, batches(2))
    assert torch.equal(m.model.embed_tokens.weight.detach(), emb_before)
    embed_unit = next(u for u in e.units if u.name == "embed")
    assert embed_unit.master is None


def test_engine_checkpoint_roundtrip(tmp_path):
    data = batches(4)
    a = make_engine(make_model(), 2)
    run(a, data[:2])
    a.save_checkpoint(tmp_path, tag="t", client_state={"hello": 1})
    rest_a = run(a, data[2:])
    b = make_engine(make_model(seed=123), 2)
    path, cs = b.load_checkpoint(tmp_path)
    assert cs == {"hello": 1} and b.global_steps == 2
    rest_b = run(b, data[2:])
    assert rest_b == rest_a
    pa, pb = full_params(a), full_params(b)
    assert all(torch.equal(pa[n], pb[n]) for n in pa)


def test_inference_engine_stage3_matches_plain_forward():
    m = make_model()
    for p in m.parameters():
        p.requires_grad_(False)
    m.eval()
    ref_out = copy.deepcopy(m)(input_ids=torch.arange(8, 40).unsqueeze(0), return_logits=True).logits
    e = TrainingEngine(m, None, None, {"zero_optimization": {"stage": 3}}, training=False)
    with torch.no_grad():
        out = e(input_ids=torch.arange(8, 40).unsqueeze(0), return_logits=True).logits
    assert torch.allclose(out, ref_out, atol=1e-5)
    # in a group of one rank nothing is gathered or released: the shard is the unit
    assert all(u.persistent for u in e.units)


def test_auto_keep_policy_follows_measured_memory(monkeypatch):
    """The memory-driven choice of layers that keep activations, driven with a fake allocator: two measuring steps
    (one layer kept), then as many layers as fit under the limit next to the measured head-room."""
    engine = make_engine(make_model(), 3, keep="auto")
    GiB = 1 << 30
    mem = {"alloc": 100 * GiB, "peak": 100 * GiB}
    monkeypatch.setattr(torch.cuda, "memory_allocated", lambda *_: mem["alloc"])
    monkeypatch.setattr(torch.cuda, "max_memory_allocated", lambda *_: mem["peak"])
    monkeypatch.setattr(torch.cuda, "memory_reserved", lambda *_: mem["alloc"])
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda *_: (180 * GiB - mem["alloc"], 180 * GiB))
    monkeypatch.setattr(torch.cuda, "reset_peak_memory_stats", lambda *_: None)
    engine.on_gpu = True
    units = engine._wrapped_units
    xs = torch.zeros(1, 1024, 64)

    def one_step(per_layer, transient=6 * GiB):
        mem["alloc"] = 100 * GiB
        kept = []
        for u in units:
            k = engine._keeps_activations(u, xs)
            kept.append(k)
            if k:
                mem["alloc"] += per_layer
        mem["peak"] = mem["alloc"] + transient
        engine._update_keep_state()
        return kept

    st = engine._keep_state
    assert one_step(4 * GiB) == [True] + [False] * (len(units) - 1) and st["phase"] == 1
    st["bytes_per_token"] = 30 * GiB / 1024  # what _run_kept would measure on the first layer
    assert one_step(30 * GiB) == [True] + [False] * (len(units) - 1) and st["phase"] == 2
    assert st["reserve"] == 36 * GiB  # one kept layer + transient: errs on the safe side
    assert st["limit"] == int(0.88 * 180 * GiB)
    # 100 + 30 (i + 1) + 36 GiB must stay under 158.4 GiB: not even the first layer fits
    assert one_step(30 * GiB) == [False] * len(units)
    st["bytes_per_token"] = 4 * GiB / 1024
    st["reserve"] = 10 * GiB
    kept = one_step(4 * GiB)
    assert kept == [100 + 4 * (i + 1) + 10 <= st["limit"] / GiB for i in range(len(units))] and all(kept)
    engine.on_gpu = False


def test_fused_reduce_decision_is_the_same_for_every_rank_of_a_partly_frozen_unit():
    """A unit whose trainable prefix is shorter than one shard (LoRA, SwiftKV-style partial freezing): the ranks
    behind the frozen tail hold no trainable element, yet they must take the same communication path."""
    from types import SimpleNamespace

    m = make_model()
    layer = m.model.layers[1]
    for n, p in layer.named_parameters():
        p.requires_grad_("input_layernorm" in n)  # only a 64-element vector trains in this layer
    e = make_engine(m, 2)
    u = next(u for u in e.units if u.name.endswith("1") and u.checkpointed)
    assert 0 < u.n_train < 256
    # pretend to be each rank of a 4-way group with the peer-memory path available
    decisions, single, lengths = [], [], []
    for r in range(4):
        u.group_size, u.group_rank, u.shard_size, u.dtype = 4, r, u.numel // 4, torch.bfloat16
        e.symm, e._grad_symm = SimpleNamespace(), [object()]
        lengths.append(u.train_len)
        decisions.append(e._fused_reduce_ok(u))
        e.cfg.gradient_clipping = 0.0
        single.append(e._single_pass_update_ok(u))
        e.cfg.gradient_clipping = 1.0
    assert lengths[0] > 0 and lengths[-1] == 0  # the premise: the local trainable length differs between ranks
    assert len(set(decisions)) == 1 and decisions[0] is True
    assert len(set(single)) == 1
    # the runs that any rank computes for a peer are that peer's own runs
    u.group_rank = 0
    assert e._runs_of_rank(u, 0) and not e._runs_of_rank(u, 3)


def test_step_raises_on_a_recorded_kernel_error_and_applies_no_update():
    from arctictraining_b200.exceptions import CommTimeoutError
    from arctictraining_b200.exceptions import KernelWaitError

    m = make_model()
    e = make_engine(m, 1)
    b = batches(1)[0]
    for words, exc in (((0, 0x102), CommTimeoutError), ((0x2801, 0), KernelWaitError), ((0, 0x3102), RuntimeError)):
        e._read_error_words = lambda w=words: w
        before = full_params(e)
        masters = [u.master.clone() for u in e.units if u.master is not None]
        out = e(**b)
        e.backward(out.loss)
        with pytest.raises(exc):
            e.step()
        assert e.global_steps == 0
        after = full_params(e)
        assert all(torch.equal(before[n], after[n]) for n in before)
        assert all(torch.equal(a, u.master) for a, u in zip(masters, [u for u in e.units if u.master is not None]))
        e.micro_steps = 0
        for u in e.units:
            u.grad_acc_valid = False


def _engine_with(model, zero_cfg, opt_cls=FusedAdamW, **extra):
    model.activation_checkpointing = True
    groups = OptimizerFactory.get_optimizer_grouped_params(model, 0.1)
    opt = opt_cls(groups, lr=1e-2, betas=(0.9, 0.95))
    return TrainingEngine(model, opt, None, {"zero_optimization": zero_cfg, "gradient_clipping": 1.0, **extra})


@pytest.mark.parametrize("ratio", [1.0, 0.5])
def test_optimizer_offload_places_units_by_ratio_and_matches_the_plain_engine(ratio):
    """``offload_optimizer`` (with ``ratio``) changes where states live, not what is computed."""
    from arctictraining_b200.optimizer.adam import CPUAdamW

    data = batches(3)
    base = _engine_with(make_model(), {"stage": 3})
    off = _engine_with(make_model(), {"stage": 3, "offload_optimizer": {"device": "cpu", "ratio": ratio}}, CPUAdamW)
    hosted = [u for u in off.units if u.host_states]
    trainable = [u for u in off.units if u.n_train > 0]
    assert hosted and (len(hosted) == len(trainable)) == (ratio == 1.0)
    frac = sum(u.n_train for u in hosted) / sum(u.n_train for u in trainable)
    assert frac >= ratio - 1e-9 and (ratio == 1.0 or frac < 1.0)
    assert not any(u.host_states for u in base.units)
    assert run(base, data) == run(off, data)
    a, b = full_params(base), full_params(off)
    assert all(torch.equal(a[n], b[n]) for n in a)


def test_offload_keys_are_read_from_the_recipe_spelling():
    from arctictraining_b200.engine.config import EngineConfig

    c = EngineConfig.from_dict({"zero_optimization": {"stage": 3, "offload_optimizer": {"device": "cpu", "ratio": 0.7},
                                                      "offload_param": {"device": "cpu"}}})
    assert c.offload_optimizer and c.offload_param and c.offload_optimizer_ratio == 0.7


def test_fp16_loss_scaling_skips_an_overflowing_step_and_halves_the_scale():
    m = make_model()
    m.activation_checkpointing = True
    groups = OptimizerFactory.get_optimizer_grouped_params(m, 0.1)
    e = TrainingEngine(m, FusedAdamW(groups, lr=1e-2), None, {
        "zero_optimization": {"stage": 1}, "gradient_clipping": 1.0,
        "fp16": {"enabled": True, "initial_scale_power": 4, "loss_scale_window": 2},
    })
    assert e.loss_scale == 16.0
    b = batches(1)[0]
    ref = make_engine(make_model(), 1)
    # good steps: same results as without scaling (the scale is divided out), scale doubles after the window
    for _ in range(2):
        la = run(e, [b])
        lb = run(ref, [b])
        assert la == pytest.approx(lb, rel=1e-5)
    assert e.loss_scale == 32.0 and e.skipped_steps == 0
    a, r = full_params(e), full_params(ref)
    assert all(torch.allclose(a[n], r[n], atol=2e-3) for n in a)  # Adam amplifies rounding of near-zero gradients
    # an overflow: the step is skipped, nothing moves, the scale halves
    out = e(**b)
    e.backward(out.loss * float("inf"))
    before = full_params(e)
    e.step()
    after = full_params(e)
    assert e.skipped_steps == 1 and e.loss_scale == 16.0
    assert all(torch.equal(before[n], after[n]) for n in before)


def test_communication_data_type_is_parsed_and_rejects_unknown_names():
    from arctictraining_b200.engine.config import EngineConfig

    assert EngineConfig.from_dict({"communication_data_type": "fp32"}).communication_data_type == torch.float32
    assert EngineConfig.from_dict({}).communication_data_type is None
    with pytest.raises(ValueError):
        EngineConfig.from_dict({"communication_data_type": "int8"})


def test_parameter_count_survives_the_release_of_stage3_units():
    m = make_model()
    want = sum(p.numel() for p in m.parameters())
    e = make_engine(m, 3)
    for u in e.units:  # what stage 3 does to a released unit on more than one rank
        if u.checkpointed:
            for p in u.params:
                p.data = torch.empty(0)
    from arctictraining_b200.trainer.trainer import Trainer

    assert Trainer._count_params(m)["total"] == want and m.num_parameters() == want


def test_bf16_master_weights_and_optimizer_states_train():
    """``bf16.bf16_master_weights_and_grads`` + ``bf16.bf16_optimizer_states``: 6 bytes per parameter of optimizer
    state instead of 16; the loss still goes down on a repeated batch."""
    cfg = load_arch_config("tiny-llama", {})
    m = CausalLM(cfg, dtype=torch.bfloat16)
    m.init_weights(seed=0)
    m.activation_checkpointing = True
    opt = FusedAdamW(OptimizerFactory.get_optimizer_grouped_params(m, 0.0), lr=3e-3, betas=(0.9, 0.95))
    e = TrainingEngine(m, opt, None, {"zero_optimization": {"stage": 3}, "gradient_clipping": 1.0,
                                      "bf16": {"enabled": True, "bf16_master_weights_and_grads": True, "bf16_optimizer_states": True}})
    assert all(u.master.dtype == torch.bfloat16 and u.grad_acc.dtype == torch.bfloat16 for u in e.units if u.master is not None)
    b = batches(1)[0]
    losses = run(e, [b] * 8)
    st = next(iter(opt.state.values()))
    assert st["exp_avg"].dtype == torch.bfloat16 and st["exp_avg_sq"].dtype == torch.bfloat16
    assert losses[-1] < losses[0] - 0.05


def test_checkpoint_patch_parks_inputs_and_keeps_gradients():
    """``torch.utils.checkpoint`` patched for host offload: same loss and gradients, the checkpointed regions' inputs
    went through the store (on a CPU device the store keeps them where they are)."""
    import torch.utils.checkpoint as ckpt

    from arctictraining_b200 import monkey_patches as mp

    torch.manual_seed(0)
    layers = torch.nn.ModuleList([torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.GELU()) for _ in range(3)])

    def run():
        for p in layers.parameters():
            p.grad = None
        x = torch.randn(8, 64, requires_grad=True, generator=torch.Generator().manual_seed(1))
        h = x
        for layer in layers:
            h = ckpt.checkpoint(layer, h, use_reentrant=False)
        h.square().mean().backward()
        return h.detach().clone(), x.grad.clone(), [p.grad.clone() for p in layers.parameters()]

    want = run()
    mp.monkey_patch_checkpoint_function_with_cpu_offload(min_bytes=0)
    try:
        mp.monkey_patch_checkpoint_function_with_cpu_offload(min_bytes=0)  # a second call changes nothing
        mp.stats.update(packed=0, restored=0)
        got = run()
    finally:
        mp.undo_checkpoint_patch()
    assert ckpt.checkpoint is not None and mp._original_checkpoint is None
    torch.testing.assert_close(got[0], want[0])
    torch.testing.assert_close(got[1], want[1])
    for a, b in zip(got[2], want[2]):
        torch.testing.assert_close(a, b)
    assert mp.stats["packed"] == 3 and mp.stats["restored"] == 3
    a, b = mp.noop_context_fn()
    with a, b:
        pass


def test_library_model_checkpoints_with_host_offload():
    """A Hugging Face model with gradient checkpointing pointed at the offloading checkpoint function: every decoder
    layer's input goes through the store, and the gradients match plain checkpointing."""
    from transformers import LlamaConfig
    from transformers import LlamaForCausalLM

    from arctictraining_b200 import monkey_patches as mp

    cfg = LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).train()
    ids = torch.randint(0, 128, (2, 16), generator=torch.Generator().manual_seed(2))

    def grads():
        model.zero_grad()
        model(input_ids=ids, labels=ids).loss.backward()
        return {n: p.grad.clone() for n, p in model.named_parameters()}

    model.gradient_checkpointing_enable()
    want = grads()
    assert mp.enable_host_offload_on_hf_model(model)
    mp.stats.update(packed=0, restored=0)
    old, mp.DEFAULT_MIN_BYTES = mp.DEFAULT_MIN_BYTES, 0
    try:
        got = grads()
    finally:
        mp.DEFAULT_MIN_BYTES = old
    assert mp.stats["packed"] >= 3 and mp.stats["packed"] == mp.stats["restored"]
    for n in want:
        torch.testing.assert_close(got[n], want[n], msg=lambda m, n=n: f"{n}: {m}")
    assert mp.enable_host_offload_on_hf_model(torch.nn.Linear(2, 2)) is False


def test_engine_section_keys_without_effect_are_named():
    from arctictraining_b200.engine.config import EngineConfig
    from arctictraining_b200.engine.config import keys_without_effect

    quiet = {"zero_optimization": {"stage": 3, "stage3_param_persistence_threshold": 10, "reduce_bucket_size": 5,
                                   "stage3_max_live_parameters": 7, "offload_optimizer": {"device": "cpu"}},
             "steps_per_print": 10, "prescale_gradients": False, "gradient_clipping": 1.0,
             "seq_parallel_communication_data_type": "bf16", "bf16": {"enabled": True}}
    assert keys_without_effect(quiet) == []
    noisy = dict(quiet, prescale_gradients=True, zero_allow_untested_optimizer=True,
                 seq_parallel_communication_data_type="fp32")
    noisy["zero_optimization"] = dict(quiet["zero_optimization"], overlap_comm=True, memory_efficient_linear=True)
    assert keys_without_effect(noisy) == ["prescale_gradients", "seq_parallel_communication_data_type",
                                          "zero_allow_untested_optimizer", "zero_optimization.memory_efficient_linear",
                                          "zero_optimization.overlap_comm"]
    assert EngineConfig.from_dict(noisy).zero_stage == 3  # reported, not refused


def test_tiled_mlp_patch_on_a_library_model_keeps_outputs_and_gradients():
    """``tiled_mlp_compute`` on a transformers model: every ``*MLP`` module runs over sequence tiles (tokens / hidden
    tiles, here 4), recomputing each tile in backward; loss and gradients are those of the plain model."""
    from transformers import LlamaConfig
    from transformers import LlamaForCausalLM

    from arctictraining_b200.ops.tiled import enable_tiled_mlp_compute
    from arctictraining_b200.ops.tiled import num_mlp_tiles

    cfg = LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg)
    ids = torch.randint(0, 128, (1, 100), generator=torch.Generator().manual_seed(3))
    assert num_mlp_tiles(torch.empty(1, 100, 32)) == 4

    def run():
        model.zero_grad()
        out = model(input_ids=ids, labels=ids)
        out.loss.backward()
        return out.loss.detach().clone(), {n: p.grad.clone() for n, p in model.named_parameters()}

    want_loss, want = run()
    assert enable_tiled_mlp_compute(model) == 2
    assert enable_tiled_mlp_compute(model) == 0  # already patched
    got_loss, got = run()
    torch.testing.assert_close(got_loss, want_loss)
    for n in want:
        torch.testing.assert_close(got[n], want[n], rtol=1e-4, atol=1e-6, msg=lambda m, n=n: f"{n}: {m}")
