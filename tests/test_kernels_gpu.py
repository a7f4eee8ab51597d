# SPDX-License-Identifier: Apache-2.0
"""Numerics of every CUDA kernel against a plain PyTorch fp32 reference of the same op."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k():
    from arctictraining_b200.ops import _ext

    _ext.require()
    return torch.ops.atb200


def _check_flag(x):
    assert int(torch.ops.atb200.read_and_clear_error_flag(x)) == 0


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("T,H", [(7, 64), (513, 4096), (33, 2048), (5, 8192)])
def test_rmsnorm_fwd_bwd(k, T, H):
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    y, rstd = k.rmsnorm_fwd(x, w, 1e-5)
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    yr = ref.rms_norm(xr, wr, 1e-5)
    yr.backward(dy.float())
    assert _rel(y, yr) < 1e-2
    dx, dw = k.rmsnorm_bwd(dy, x, w, rstd)
    assert _rel(dx, xr.grad) < 1e-2
    assert _rel(dw, wr.grad) < 1e-2


def test_rope_matches_reference_and_inverts(k):
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    T, Hq, Hkv, D = 300, 8, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    pos = torch.arange(T, device="cuda").unsqueeze(0)
    cos, sin = ref.rope_cos_sin(pos, D, 500000.0)
    q_ref = ref.rope_apply(qkv[:, : Hq * D].reshape(1, T, Hq, D), cos, sin)
    orig = qkv.clone()
    k.rope_inplace(qkv[:, : Hq * D].unflatten(1, (Hq, D)), cos[0].contiguous(), sin[0].contiguous(), False)
    assert _rel(qkv[:, : Hq * D].reshape(1, T, Hq, D), q_ref) < 1e-2
    assert torch.equal(qkv[:, Hq * D :], orig[:, Hq * D :])  # k and v untouched by this call
    k.rope_inplace(qkv[:, : Hq * D].unflatten(1, (Hq, D)), cos[0].contiguous(), sin[0].contiguous(), True)
    assert _rel(qkv, orig) < 2e-2


def test_swiglu_fwd_bwd(k):
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    T, I = 257, 1536
    gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    out = k.swiglu_fwd(gu)
    gr = gu.float().requires_grad_(True)
    o_ref = ref.swiglu_interleaved(gr)
    o_ref.backward(dout.float())
    assert _rel(out, o_ref) < 1e-2
    assert _rel(k.swiglu_bwd(dout, gu), gr.grad) < 1e-2


@pytest.mark.parametrize("n", [1024, 4099, 1 << 20])
def test_adamw_matches_torch(k, n):
    torch.manual_seed(0)
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16) if n % 4 == 0 else None
    pr = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    scale = torch.tensor([0.5], device="cuda")
    for step in range(1, 4):
        pr.grad = g * 0.5
        opt.step()
        k.adamw_step(p, g, m, v, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, scale)
    assert _rel(p, pr.detach()) < 1e-5
    if lp is not None:
        assert _rel(lp, p) < 5e-3


def test_sumsq_and_accum(k):
    torch.manual_seed(0)
    x = torch.randn(1 << 20, device="cuda")
    assert abs(float(k.sumsq(x)) - float(x.double().pow(2).sum())) / float(x.double().pow(2).sum()) < 1e-5
    src = torch.randn(10007 * 8, device="cuda", dtype=torch.bfloat16)
    acc = torch.ones(10007 * 8, device="cuda")
    k.accum_bf16(src, acc, 0.25, False)
    assert _rel(acc, 1 + 0.25 * src.float()) < 1e-6
    k.accum_bf16(src, acc, 2.0, True)
    assert _rel(acc, 2.0 * src.float()) < 1e-6


@pytest.mark.parametrize("T,V", [(9, 1024), (130, 32000), (17, 128256)])
def test_cross_entropy_kernel(k, T, V):
    torch.manual_seed(0)
    logits = (3 * torch.randn(T, V, device="cuda")).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::4] = -100
    lr = logits.float().requires_grad_(True)
    loss_ref = torch.nn.functional.cross_entropy(lr, labels, ignore_index=-100, reduction="sum")
    loss_ref.backward()
    scale = torch.tensor([0.5], device="cuda")
    work = logits.clone()
    loss, lse = k.ce_fwd_bwd(work, labels, scale, None, True)
    assert abs(float(loss.sum()) - float(loss_ref)) / float(loss_ref) < 2e-3
    assert _rel(work, 0.5 * lr.grad) < 2e-2
    assert torch.all(work[::4] == 0)


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (300, 264, 200), (1024, 4096, 4096), (8, 8, 8), (4096, 1024, 8192), (520, 1032, 72)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_tn(k, M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = k.gemm_bf16(a, b, False, False, 0, None, 0)
    torch.cuda.synchronize()
    _check_flag(a)
    ref = a.float() @ b.float().t()
    assert _rel(c, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (304, 264, 200), (1024, 2048, 4096)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
def test_gemm_mn_major_operands(k, M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16) if a_mn else torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16) if b_mn else torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = k.gemm_bf16(a, b, a_mn, b_mn, 0, None, 0)
    torch.cuda.synchronize()
    _check_flag(a)
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    assert _rel(c, af @ bf) < 1e-2


def test_gemm_accumulate_and_swiglu_epilogues(k):
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    M, N, K = 384, 768, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (0.1 * torch.randn(N, K, device="cuda")).bfloat16()
    base = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out = base.clone()
    k.gemm_bf16(a, b, False, False, 1, out, 0)
    assert _rel(out, base.float() + a.float() @ b.float().t()) < 1e-2
    h = k.gemm_bf16(a, b, False, False, 2, None, 0)
    torch.cuda.synchronize()
    _check_flag(a)
    assert h.shape == (M, N // 2)
    assert _rel(h, ref.swiglu_interleaved(a.float() @ b.float().t())) < 1e-2


def test_gemm_is_deterministic(k):
    torch.manual_seed(0)
    a = torch.randn(1024, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(2048, 1024, device="cuda", dtype=torch.bfloat16)
    c1 = k.gemm_bf16(a, b, False, False, 0, None, 0)
    c2 = k.gemm_bf16(a, b, False, False, 0, None, 0)
    assert torch.equal(c1, c2)


def test_linear_autograd_matches_torch():
    from arctictraining_b200 import ops

    torch.manual_seed(0)
    x = torch.randn(4, 96, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(1024, 512, device="cuda")).bfloat16().requires_grad_(True)
    y = ops.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


def test_linear_swiglu_autograd():
    from arctictraining_b200 import ops
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    x = torch.randn(200, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(1024, 256, device="cuda")).bfloat16().requires_grad_(True)
    h = ops.linear_swiglu(x, w)
    g = torch.randn_like(h)
    h.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    hr = ref.swiglu_interleaved(torch.nn.functional.linear(xr, wr))
    hr.backward(g.float())
    assert _rel(h, hr) < 1e-2 and _rel(x.grad, xr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 2e-2


def test_fused_linear_cross_entropy_matches_torch():
    from arctictraining_b200 import ops

    torch.manual_seed(0)
    T, H, V = 700, 256, 4096
    h = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(V, H, device="cuda")).bfloat16().requires_grad_(True)
    y = torch.randint(0, V, (T,), device="cuda")
    y[:100] = -100
    loss_sum, n = ops.fused_linear_cross_entropy(h, w, y, chunk_tokens=256)
    (loss_sum / n).backward()
    hr = h.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    lr = torch.nn.functional.cross_entropy(hr @ wr.t(), y, ignore_index=-100)
    lr.backward()
    assert abs(float(loss_sum / n) - float(lr)) < 2e-2
    assert _rel(h.grad, hr.grad) < 3e-2 and _rel(w.grad, wr.grad) < 3e-2


def test_fused_linear_logprobs_matches_torch():
    from arctictraining_b200 import ops

    torch.manual_seed(0)
    T, H, V = 300, 128, 2048
    h = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(V, H, device="cuda")).bfloat16().requires_grad_(True)
    y = torch.randint(0, V, (T,), device="cuda")
    y[::3] = -100
    lp = ops.fused_linear_logprobs(h, w, y, chunk_tokens=128)
    coef = torch.randn(T, device="cuda")
    (lp * coef).sum().backward()
    hr = h.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    lpr = torch.log_softmax(hr @ wr.t(), -1).gather(1, y.clamp(min=0).unsqueeze(1)).squeeze(1) * (y != -100)
    (lpr * coef).sum().backward()
    assert _rel(lp, lpr) < 2e-2
    assert _rel(h.grad, hr.grad) < 3e-2 and _rel(w.grad, wr.grad) < 3e-2


# ------------------------------------------------------------------------------------------------ MoE kernels
def test_moe_gating_kernel_matches_reference(k):
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    for E, K, dtype in [(128, 8, torch.bfloat16), (8, 2, torch.float32), (60, 4, torch.float32)]:
        logits = torch.randn(777, E, device="cuda", dtype=dtype)
        probs, scores, experts = k.moe_topk_gating_fwd(logits, K, True)
        p_ref, s_ref, e_ref = ref.topk_gating(logits, K, True)
        assert _rel(probs, p_ref) < 1e-5
        assert torch.equal(experts.long(), e_ref)
        assert _rel(scores, s_ref) < 1e-5


def test_moe_gating_backward_matches_autograd(k):
    torch.manual_seed(0)
    T, E, K = 300, 64, 4
    logits = torch.randn(T, E, device="cuda")
    probs, scores, experts = k.moe_topk_gating_fwd(logits, K, True)
    dscores = torch.randn(T, K, device="cuda")
    extra = torch.rand(E, device="cuda") * 0.01
    dlogits = k.moe_topk_gating_bwd(dscores, probs, experts, extra, True)
    lr = logits.clone().requires_grad_(True)
    pr = torch.softmax(lr, -1)
    sr = torch.gather(pr, 1, experts.long())
    sr = sr / sr.sum(-1, keepdim=True)
    ((sr * dscores).sum() + (pr * extra).sum()).backward()
    assert _rel(dlogits, lr.grad) < 1e-4


def test_moe_slots_scatter_gather_kernels(k):
    from arctictraining_b200.moe import ops as mops

    torch.manual_seed(0)
    T, K, E, H = 5000, 8, 128, 256
    experts = torch.randint(0, E, (T, K), device="cuda", dtype=torch.int32)
    slots, counts, offsets = k.moe_assign_slots(experts, E, 128)
    s_ref, c_ref, o_ref = mops.assign_slots(experts.cpu(), E, 128)
    assert torch.equal(slots.cpu(), s_ref) and torch.equal(counts.cpu(), c_ref) and torch.equal(offsets.cpu(), o_ref)
    rows = int(offsets[-1])
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    perm = k.moe_scatter_fwd(x, slots, rows)
    assert torch.equal(perm[slots[:, 3].long()], x)
    scores = torch.rand(T, K, device="cuda")
    out = k.moe_gather_fwd(perm, slots, scores)
    assert _rel(out, x.float() * scores.sum(-1, keepdim=True)) < 1e-2
    dout = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    dy, dscores = k.moe_gather_bwd(dout, perm, slots, scores)
    assert _rel(dscores, (dout.float() * x.float()).sum(-1, keepdim=True).expand(T, K)) < 1e-2
    assert _rel(k.moe_scatter_bwd(dy, slots), dout.float() * scores.sum(-1, keepdim=True)) < 1e-2


def test_moe_slot_assignment_and_scatter_are_bit_identical_on_a_second_run(k):
    """Slots inside an expert follow the (token, k) order — no atomics decide them — so slot maps, permuted rows, the
    combine and its gradients repeat bit for bit; rows of the permuted buffer that belong to no token stay zero."""
    torch.manual_seed(2)
    T, K, E, H = 3001, 4, 64, 128
    experts = torch.randint(0, E, (T, K), device="cuda", dtype=torch.int32)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    scores = torch.rand(T, K, device="cuda")
    dout = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    runs = []
    for _ in range(2):
        slots, counts, offsets = k.moe_assign_slots(experts, E, 128)
        rows = int(offsets[-1])
        perm = k.moe_scatter_fwd(x, slots, rows)
        out = k.moe_gather_fwd(perm, slots, scores)
        dy, dscores = k.moe_gather_bwd(dout, perm, slots, scores)
        dx = k.moe_scatter_bwd(dy, slots)
        runs.append((slots, counts, offsets, perm, out, dy, dscores, dx))
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    slots, _, offsets, perm = runs[0][:4]
    used = torch.zeros(int(offsets[-1]), dtype=torch.bool, device="cuda")
    used[slots.reshape(-1).long()] = True
    assert int(used.sum()) == T * K and not bool(perm[~used].any())


def test_grouped_mlp_matches_reference_forward_and_backward(k):
    from arctictraining_b200.moe import ops as mops
    from arctictraining_b200.moe.grouped import grouped_mlp_reference
    from arctictraining_b200.moe.grouped_cuda import grouped_mlp_cuda

    torch.manual_seed(0)
    E, H, I, T, K = 6, 256, 192, 900, 2
    experts = torch.randint(0, E - 1, (T, K), device="cuda", dtype=torch.int32)  # the last expert stays empty
    slots, counts, offsets = k.moe_assign_slots(experts, E, 128)
    rows = T * K + E * 127
    rows = (rows + 127) // 128 * 128
    x = (0.5 * torch.randn(T, H, device="cuda")).bfloat16()
    perm = k.moe_scatter_fwd(x, slots, rows).requires_grad_(True)
    wgu = (0.05 * torch.randn(E, 2 * I, H, device="cuda")).bfloat16().requires_grad_(True)
    wd = (0.05 * torch.randn(E, H, I, device="cuda")).bfloat16().requires_grad_(True)
    y = grouped_mlp_cuda(perm, offsets, wgu, wd)
    with torch.no_grad():
        y_nograd = grouped_mlp_cuda(perm.detach(), offsets, wgu.detach(), wd.detach())
    g = torch.randn_like(y)
    used = torch.zeros(rows, 1, device="cuda")
    used[slots.reshape(-1).long()] = 1
    g = (g * used).bfloat16()  # gradients of padding rows are zero in the real layer
    y.backward(g)
    torch.cuda.synchronize()
    _check_flag(x)
    pr = perm.detach().float().requires_grad_(True)
    wgur = wgu.detach().float().requires_grad_(True)
    wdr = wd.detach().float().requires_grad_(True)
    yr = grouped_mlp_reference(pr, offsets, wgur, wdr)
    yr.backward(g.float())
    assert _rel(y, yr) < 2e-2 and _rel(y_nograd, yr) < 2e-2
    assert _rel(perm.grad, pr.grad) < 3e-2
    assert _rel(wgu.grad, wgur.grad) < 3e-2 and _rel(wd.grad, wdr.grad) < 3e-2
    assert float(wgu.grad[E - 1].abs().max()) == 0.0


def test_arctic_moe_layer_on_gpu_matches_cpu_reference():
    from arctictraining_b200.moe.layer import ArcticMoE
    from arctictraining_b200.moe.layer import MoEConfig

    torch.manual_seed(0)
    cfgd = dict(model_dim=256, intermediate_dim=128, num_experts=16, top_k=4, loss_coeff=0.01)
    cpu = ArcticMoE(MoEConfig(**cfgd), dtype=torch.float32)
    for p in cpu.parameters():
        torch.nn.init.normal_(p, std=0.08)
    gpu = ArcticMoE(MoEConfig(**cfgd), dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        for a, b in zip(gpu.parameters(), cpu.parameters()):
            a.copy_(b)
            b.copy_(a.float().cpu())  # same bf16-rounded weights on both sides
    x = torch.randn(500, 256)
    xg = x.cuda().bfloat16().requires_grad_(True)
    xc = xg.detach().float().cpu().requires_grad_(True)
    yg, yc = gpu(xg), cpu(xc)
    yg.float().pow(2).sum().backward()
    yc.pow(2).sum().backward()
    assert _rel(yg.cpu(), yc) < 3e-2
    assert _rel(xg.grad.cpu(), xc.grad) < 5e-2
    assert _rel(gpu.expert_down.grad.cpu(), cpu.expert_down.grad) < 5e-2
    assert _rel(gpu.router_gate.grad.cpu(), cpu.router_gate.grad) < 8e-2


# ------------------------------------------------------------------------------------------------ CTA-pair GEMM
@pytest.fixture
def cta_pairs(k):
    old = k.set_gemm_cta_pairs(True)
    yield
    k.set_gemm_cta_pairs(old)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (300, 264, 200), (8, 8, 8), (4096, 1024, 4096), (1000, 520, 72)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_cta_pair_kernel(k, cta_pairs, M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    if a_mn and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    a = torch.randn(K, M, device="cuda", dtype=torch.bfloat16) if a_mn else torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16) if b_mn else torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = k.gemm_bf16(a, b, a_mn, b_mn, 0, None, 0)
    torch.cuda.synchronize()
    _check_flag(a)
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    assert _rel(c, af @ bf) < 1e-2


def test_gemm_cta_pair_epilogues(k, cta_pairs):
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    M, N, K = 640, 1024, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (0.1 * torch.randn(N, K, device="cuda")).bfloat16()
    base = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out = base.clone()
    k.gemm_bf16(a, b, False, False, 1, out, 0)
    assert _rel(out, base.float() + a.float() @ b.float().t()) < 1e-2
    h = k.gemm_bf16(a, b, False, False, 2, None, 0)
    torch.cuda.synchronize()
    _check_flag(a)
    assert _rel(h, ref.swiglu_interleaved(a.float() @ b.float().t())) < 1e-2


@pytest.mark.parametrize(
    "lens,Hq,Hkv",
    [([256], 4, 4), ([128, 384], 8, 2), ([100, 37, 411, 129], 4, 1), ([1000], 2, 2), ([1, 127, 128, 129], 4, 2)],
)
def test_native_flash_attention_forward(k, lens, Hq, Hkv):
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : Hq * 128].view(T, Hq, 128)          # strided views of one fused projection output
    kk = qkv[:, Hq * 128 : (Hq + Hkv) * 128].view(T, Hkv, 128)
    v = qkv[:, (Hq + Hkv) * 128 :].view(T, Hkv, 128)
    scale = 128 ** -0.5
    out, lse = k.fmha_fwd(q, kk, v, cu, T // 128 + len(lens), scale)
    assert k.read_and_clear_error_flag(out) == 0
    want = ref.attention(q[None], kk[None], v[None], cu_seqlens=cu.long(), scale=scale)[0]
    torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)
    # log-sum-exp against fp32 scores
    qf = q.float().transpose(0, 1)
    kf = kk.float().transpose(0, 1).repeat_interleave(Hq // Hkv, dim=0)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    seg = ref.segment_ids_from_cu(cu.long(), T)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool, device="cuda")) & (seg[:, None] == seg[None, :])
    want_lse = torch.logsumexp(s.masked_fill(~mask, float("-inf")), dim=-1)
    torch.testing.assert_close(lse, want_lse, atol=1e-2, rtol=1e-3)


def test_native_attention_autograd_matches_reference():
    from arctictraining_b200.ops import functional as Fn
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(1)
    S, Hq, Hkv = 640, 4, 2
    cu = torch.tensor([0, 200, 640], device="cuda", dtype=torch.int32)
    q = torch.randn(1, S, Hq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    kk = torch.randn(1, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(1, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(1, S, Hq, 128, device="cuda", dtype=torch.bfloat16)
    o = Fn.attention(q, kk, v, cu_seqlens=cu, max_seqlen=440, impl="native")
    o.backward(g)
    got = [o, q.grad, kk.grad, v.grad]
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, kk, v))
    o2 = ref.attention(qr, kr, vr, cu_seqlens=cu.long())
    o2.backward(g.float())
    for a, b in zip(got, [o2, qr.grad, kr.grad, vr.grad]):
        torch.testing.assert_close(a.float(), b.float(), atol=5e-2, rtol=5e-2)
    # batch of equal-length rows without cu_seqlens
    q2 = torch.randn(2, 256, Hq, 128, device="cuda", dtype=torch.bfloat16)
    k2 = torch.randn(2, 256, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    v2 = torch.randn(2, 256, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    torch.testing.assert_close(
        Fn.attention(q2, k2, v2, impl="native").float(), ref.attention(q2, k2, v2).float(), atol=2e-2, rtol=2e-2
    )


def test_linear_with_fused_residual_matches_torch():
    from arctictraining_b200.ops import functional as Fn

    torch.manual_seed(0)
    x = (torch.randn(2, 192, 256, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    r = torch.randn(2, 192, 512, device="cuda").bfloat16().requires_grad_(True)
    g = torch.randn(2, 192, 512, device="cuda").bfloat16()
    y = Fn.linear(x, w, None, r)
    y.backward(g)
    xr, wr, rr = (t.detach().float().requires_grad_(True) for t in (x, w, r))
    y2 = rr + xr @ wr.t()
    y2.backward(g.float())
    assert _rel(y, y2) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2
    assert torch.equal(r.grad, g)
    _check_flag(y)


@pytest.mark.parametrize("with_residual", [False, True])
def test_fused_mlp_function_matches_reference(with_residual):
    from arctictraining_b200.ops import functional as Fn
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(0)
    H, I, T = 256, 384, 320
    x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    wgu = (torch.randn(2 * I, H, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    wd = (torch.randn(H, I, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    r = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True) if with_residual else None
    g = torch.randn(T, H, device="cuda").bfloat16()
    y = Fn.mlp_swiglu(x, wgu, wd, r)
    y.backward(g)
    xr, wgur, wdr = (t.detach().float().requires_grad_(True) for t in (x, wgu, wd))
    y2 = ref.swiglu_interleaved(xr @ wgur.t()) @ wdr.t()
    if with_residual:
        y2 = y2 + r.detach().float()
    y2.backward(g.float())
    assert _rel(y, y2) < 1e-2
    for a, b in ((x.grad, xr.grad), (wgu.grad, wgur.grad), (wd.grad, wdr.grad)):
        assert _rel(a, b) < 1.5e-2
    if with_residual:
        assert torch.equal(r.grad, g)
    _check_flag(y)


def test_weight_gradient_accumulates_into_the_engine_buffer():
    from arctictraining_b200.ops import functional as Fn

    torch.manual_seed(0)
    x = (torch.randn(256, 128, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(192, 128, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    g = torch.randn(256, 192, device="cuda").bfloat16()
    Fn.linear(x, w).backward(g)
    want = w.grad.clone()
    w.grad = None
    main = torch.ones_like(w)
    w._atb_main_grad = main
    Fn.linear(x, w).backward(g)
    assert w.grad is None
    assert _rel(main - 1, want) < 1e-2


def test_argument_errors_raise_with_a_readable_message(k):
    a = torch.randn(128, 64, device="cuda").bfloat16()
    b = torch.randn(128, 64, device="cuda").bfloat16()
    with pytest.raises(RuntimeError, match="unsupported epilogue 7"):
        k.gemm_bf16(a, b, False, False, 7, None, 0, None)
    with pytest.raises(RuntimeError, match="head_dim must be 128"):
        k.fmha_fwd(a.view(128, 1, 64), b.view(128, 1, 64), b.view(128, 1, 64), torch.tensor([0, 128], device="cuda", dtype=torch.int32), 2, 0.1)


def test_native_attention_dense_backward_matches_reference():
    """Unpacked sequences (a batch of rows, strided views of a fused projection) through the autograd function."""
    from arctictraining_b200.ops import functional as Fn
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(2)
    B, S, Hq, Hkv = 2, 384, 4, 2
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    q, kk, v = qkv.view(B, S, Hq + 2 * Hkv, 128).split([Hq, Hkv, Hkv], dim=2)  # strided views of a fused buffer
    g = torch.randn(B, S, Hq, 128, device="cuda", dtype=torch.bfloat16)
    o = Fn.attention(q, kk, v, impl="native")
    o.backward(g)
    x2 = qkv.detach().float().requires_grad_(True)
    q2, k2, v2 = x2.view(B, S, Hq + 2 * Hkv, 128).split([Hq, Hkv, Hkv], dim=2)
    o2 = ref.attention(q2, k2, v2)
    o2.backward(g.float())
    assert _rel(o, o2) < 1e-2
    assert _rel(qkv.grad, x2.grad) < 2e-2


def _attention_grads_fp32_chunked(q, kk, v, g, scale, chunk=4096):
    """fp32 causal attention (one unpacked sequence) with its gradients, query chunk by query chunk, so that a long
    sequence never needs the full score matrix.  q / g [T, Hq, D], kk / v [T, Hkv, D].  Returns (o, lse, dq, dk, dv)."""
    T, Hq, D = q.shape
    Hkv = kk.shape[1]
    o = torch.empty(T, Hq, D, device=q.device)
    lse = torch.empty(Hq, T, device=q.device)
    dq = torch.empty(T, Hq, D, device=q.device)
    dk = torch.zeros(T, Hkv, D, device=q.device)
    dv = torch.zeros(T, Hkv, D, device=q.device)
    pos = torch.arange(T, device=q.device)
    for h in range(Hq):
        hk = h // (Hq // Hkv)
        kf, vf = kk[:, hk].float(), v[:, hk].float()
        for a in range(0, T, chunk):
            b = min(T, a + chunk)
            qf, gf = q[a:b, h].float(), g[a:b, h].float()
            s = (qf @ kf[:b].t()) * scale
            s.masked_fill_(pos[None, :b] > pos[a:b, None], float("-inf"))
            l = torch.logsumexp(s, dim=-1)
            p = torch.exp(s - l[:, None])
            oc = p @ vf[:b]
            dp = gf @ vf[:b].t()
            ds = p * (dp - (gf * oc).sum(-1, keepdim=True))
            o[a:b, h], lse[h, a:b] = oc, l
            dq[a:b, h] = (ds @ kf[:b]) * scale
            dk[:b, hk] += (ds.t() @ qf) * scale
            dv[:b, hk] += p.t() @ gf
    return o, lse, dq, dk, dv


@pytest.mark.parametrize(
    "lens,Hq,Hkv",
    [([256], 4, 4), ([128, 384], 8, 2), ([100, 37, 411, 129], 4, 1), ([1000], 2, 2), ([1, 127, 128, 129], 4, 2),
     ([2048, 700], 8, 2)],
)
def test_native_flash_attention_backward(k, lens, Hq, Hkv):
    """dq / dk / dv of the tcgen05 backward kernel against fp32 autograd of the reference attention."""
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(3)
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : Hq * 128].view(T, Hq, 128)          # strided views of one fused projection output
    kk = qkv[:, Hq * 128 : (Hq + Hkv) * 128].view(T, Hkv, 128)
    v = qkv[:, (Hq + Hkv) * 128 :].view(T, Hkv, 128)
    g = torch.randn(T, Hq, 128, device="cuda", dtype=torch.bfloat16)
    scale = 128 ** -0.5
    nblk = T // 128 + len(lens)
    out, lse = k.fmha_fwd(q, kk, v, cu, nblk, scale)
    dq, dk, dv = k.fmha_bwd(g, q, kk, v, out, lse, cu, nblk, scale)
    torch.cuda.synchronize()
    _check_flag(out)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, kk, v))
    o2 = ref.attention(qr[None], kr[None], vr[None], cu_seqlens=cu.long(), scale=scale)[0]
    o2.backward(g.float())
    for name, a, b in (("dq", dq, qr.grad), ("dk", dk, kr.grad), ("dv", dv, vr.grad)):
        assert torch.isfinite(a.float()).all(), name
        assert _rel(a, b) < 2e-2, (name, _rel(a, b))
        torch.testing.assert_close(a.float(), b, atol=6e-2, rtol=6e-2, msg=lambda m: f"{name}: {m}")
    # dk and dv are accumulated in a fixed order: bit-identical on a second run; dq to fp32 rounding of its sum
    dq2, dk2, dv2 = k.fmha_bwd(g, q, kk, v, out, lse, cu, nblk, scale)
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)
    torch.testing.assert_close(dq2.float(), dq.float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("lens,Hq,Hkv", [([384], 4, 2), ([200, 56, 512], 8, 2)])
def test_rope_attention_fused_node_matches_fp32_reference(k, lens, Hq, Hkv):
    """Rotary embedding + attention on a fused projection output as one autograd node: output and the gradient of the
    projection (one tensor, written by the backward kernel without concatenation) against fp32 autograd of
    rope -> attention; the packed form of the backward kernel equals its three-tensor form bit for bit."""
    from arctictraining_b200 import ops
    from arctictraining_b200.ops import reference as ref

    torch.manual_seed(11)
    T, D = sum(lens), 128
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens]).cuda()[None]
    cos, sin = ref.rope_cos_sin(pos, D, 10000.0)
    base = torch.randn(1, T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(1, T, Hq, D, device="cuda", dtype=torch.bfloat16)

    src = base.clone().requires_grad_(True)
    out = ops.rope_attention(src * 1, cos, sin, Hq, Hkv, D, cu, max(lens))  # "* 1": a non-leaf, as a projection output is
    assert out is not None
    out.backward(g)
    torch.cuda.synchronize()
    _check_flag(out)

    x = base.float().detach().requires_grad_(True)
    q, kk, v = x.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    qr = ref.rope_apply(q.view(1, T, Hq, D), cos, sin)
    kr = ref.rope_apply(kk.view(1, T, Hkv, D), cos, sin)
    o2 = ref.attention(qr, kr, v.view(1, T, Hkv, D), cu_seqlens=cu.long())
    o2.backward(g.float())
    assert _rel(out, o2) < 1e-2
    assert _rel(src.grad, x.grad) < 2e-2, _rel(src.grad, x.grad)
    for lo, hi, name in ((0, Hq * D, "dq"), (Hq * D, (Hq + Hkv) * D, "dk"), ((Hq + Hkv) * D, (Hq + 2 * Hkv) * D, "dv")):
        assert _rel(src.grad[..., lo:hi], x.grad[..., lo:hi]) < 2e-2, name

    # packed and three-tensor forms of the backward kernel agree exactly (dk, dv) / to fp32 summation order (dq)
    qkv = base[0].clone()
    qv = qkv[:, : Hq * D].view(T, Hq, D)
    kv_ = qkv[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    vv = qkv[:, (Hq + Hkv) * D :].view(T, Hkv, D)
    nblk = T // 128 + len(lens)
    o, lse = k.fmha_fwd(qv, kv_, vv, cu, nblk, D ** -0.5)
    a = k.fmha_bwd(g[0], qv, kv_, vv, o, lse, cu, nblk, D ** -0.5)
    b = k.fmha_bwd(g[0], qv, kv_, vv, o, lse, cu, nblk, D ** -0.5, True)
    assert b[0].stride(0) == (Hq + 2 * Hkv) * D and b[1].data_ptr() == b[0].data_ptr() + Hq * D * 2
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    torch.testing.assert_close(a[0].float(), b[0].float(), atol=1e-2, rtol=1e-2)


def test_native_flash_attention_long_sequence_forward_and_backward(k):
    """65 536 tokens (64-bit offsets, log-sum-exp layout, 512 key blocks) against a chunked fp32 reference."""
    torch.manual_seed(4)
    T, Hq, Hkv = 65536, 2, 1
    q = torch.randn(T, Hq, 128, device="cuda", dtype=torch.bfloat16)
    kk = torch.randn(T, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(T, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(T, Hq, 128, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0, T], device="cuda", dtype=torch.int32)
    scale = 128 ** -0.5
    out, lse = k.fmha_fwd(q, kk, v, cu, T // 128 + 1, scale)
    dq, dk, dv = k.fmha_bwd(g, q, kk, v, out, lse, cu, T // 128 + 1, scale)
    torch.cuda.synchronize()
    _check_flag(out)
    o2, lse2, dq2, dk2, dv2 = _attention_grads_fp32_chunked(q, kk, v, g, scale)
    torch.testing.assert_close(lse, lse2, atol=1e-2, rtol=1e-3)
    assert _rel(out, o2) < 1e-2
    for name, a, b in (("dq", dq, dq2), ("dk", dk, dk2), ("dv", dv, dv2)):
        assert _rel(a, b) < 2e-2, (name, _rel(a, b))


def test_native_flash_attention_forward_262144_tokens_sampled_rows(k):
    """Forward at 262 144 tokens: three blocks of query rows (first, middle, last) against fp32."""
    torch.manual_seed(5)
    T = 262144
    q = torch.randn(T, 1, 128, device="cuda", dtype=torch.bfloat16)
    kk = torch.randn(T, 1, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(T, 1, 128, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0, T], device="cuda", dtype=torch.int32)
    scale = 128 ** -0.5
    out, lse = k.fmha_fwd(q, kk, v, cu, T // 128 + 1, scale)
    torch.cuda.synchronize()
    _check_flag(out)
    pos = torch.arange(T, device="cuda")
    for a in (0, T // 2 - 300, T - 1024):
        b = a + 1024
        s = (q[a:b, 0].float() @ kk[:b, 0].float().t()) * scale
        s.masked_fill_(pos[None, :b] > pos[a:b, None], float("-inf"))
        want_lse = torch.logsumexp(s, dim=-1)
        want = torch.softmax(s, dim=-1) @ v[:b, 0].float()
        torch.testing.assert_close(lse[0, a:b], want_lse, atol=1e-2, rtol=1e-3)
        assert _rel(out[a:b, 0], want) < 1e-2
