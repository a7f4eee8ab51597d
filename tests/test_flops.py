# SPDX-License-Identifier: Apache-2.0
"""Floating-point operation estimates against hand-counted values."""

from arctictraining_b200.flops import FlopsCounter


def test_dense_llama_counts_weights_and_causal_scores():
    cfg = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
               vocab_size=100)
    fc = FlopsCounter(cfg, model_size=0)
    per_layer = 64 * 128 * 3 + 64 * (64 + 2 * 32 + 64)
    weights = per_layer * 2 + 100 * 64
    expect = (6 * weights * 30 + 12 * (10 * 10 + 20 * 20) * 16 * 4 * 2) / 1e12
    assert abs(fc.estimate_tflos([10, 20]) - expect) < 1e-15
    fwd = (2 * weights * 30 + 2 * (10 * 10 + 20 * 20) * 16 * 4 * 2) / 1e12
    assert abs(fc.estimate_tflos([10, 20], forward_only=True) - fwd) < 1e-15
    ckpt = FlopsCounter(cfg, 0, enable_gradient_checkpointing=True).estimate_tflos([30])
    assert abs(ckpt - (8 * weights * 30 + 16 * 900 * 16 * 4 * 2) / 1e12) < 1e-15


def test_deepseek_mla_with_routed_and_shared_experts():
    cfg = dict(hidden_size=32, intermediate_size=64, moe_intermediate_size=16, num_hidden_layers=3, first_k_dense_replace=1,
               num_attention_heads=2, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, vocab_size=50,
               qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8, q_lora_rank=None, kv_lora_rank=12)
    attn = 32 * 2 * 12 + 32 * (12 + 4) + 2 * (8 + 8) * 12 + 2 * 8 * 32
    moe = 32 * 8 + 32 * 16 * 3 * 3
    n = (moe + attn) * 2 + (32 * 64 * 3 + attn) * 1 + 50 * 32
    expect = (6 * n * 7 + 12 * 49 * 3 * 12 * 2) / 1e12
    assert abs(FlopsCounter(cfg, 0).estimate_tflos([7]) - expect) < 1e-15
    cfg["q_lora_rank"] = 6
    attn_lr = attn - 32 * 2 * 12 + 32 * 6 + 6 * 2 * 12
    n_lr = (moe + attn_lr) * 2 + (32 * 64 * 3 + attn_lr) + 50 * 32
    assert abs(FlopsCounter(cfg, 0).estimate_tflos([7]) - (6 * n_lr * 7 + 12 * 49 * 3 * 12 * 2) / 1e12) < 1e-15


def test_hybrid_linear_attention_layers_have_no_quadratic_term():
    cfg = dict(hidden_size=32, num_hidden_layers=4, full_attention_interval=4, num_attention_heads=2, num_key_value_heads=1,
               head_dim=16, vocab_size=10, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=8,
               linear_key_head_dim=4, linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=2,
               linear_conv_kernel_dim=4)
    mlp = 32 * 2 * 8 * 3 + 32 * 4
    full = 32 * (32 + 16 + 16 + 32)
    lin = 32 * (2 * 8 + 2 * 16 + 2 * 2) + 4 * (2 * 8 + 16) + 2 * 64 * 4 + 32 * 16
    n = mlp * 4 + full * 1 + lin * 3 + 10 * 32
    expect = (6 * n * 5 + 12 * 25 * 16 * 2 * 1) / 1e12
    assert abs(FlopsCounter(cfg, 0).estimate_tflos([5]) - expect) < 1e-15
