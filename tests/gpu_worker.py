# SPDX-License-Identifier: Apache-2.0
"""Worker for the multi-GPU tests (NCCL, one process per GPU).  ``python tests/gpu_worker.py <scenario> <out_dir>``."""

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

OVERRIDES = dict(num_hidden_layers=3, hidden_size=512, intermediate_size=1024, num_attention_heads=8,
                 num_key_value_heads=2, vocab_size=4096)


def make_engine(stage, fused, seed=0, clip=1.0):
    cfg = load_arch_config("llama-3.1-8b", OVERRIDES)
    with torch.device("cuda"):
        m = CausalLM(cfg, dtype=torch.bfloat16)
    m.init_weights(seed=seed)
    m.attn_impl = "sdpa"
    opt = FusedAdamW(OptimizerFactory.get_optimizer_grouped_params(m, 0.1), lr=1e-3, betas=(0.9, 0.95))
    return TrainingEngine(m, opt, None, {"zero_optimization": {"stage": stage}, "gradient_clipping": clip,
                                         "bfloat16": {"enabled": True}, "fused_comm": "auto" if fused else "off"})


def run(engine, n=3, seed=0):
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(seed)
    losses = []
    for _ in range(n):
        ids = torch.randint(8, 4096, (world, 256), generator=g)[rank : rank + 1].cuda()
        out = engine(input_ids=ids, labels=ids.clone())
        engine.backward(out.loss)
        engine.step()
        losses.append(float(out.loss))
    torch.cuda.synchronize()
    return losses


class pytest_approx:
    def __init__(self, v, rel=2e-2):
        self.v, self.rel = v, rel

    def __eq__(self, other):
        return abs(other - self.v) <= self.rel * abs(self.v)


def scenario_fused_vs_nccl(out_dir):
    res = {}
    for stage, clip in ((2, 1.0), (3, 1.0), (3, 0.0)):
        a = make_engine(stage, fused=False, clip=clip)
        la = run(a)
        pa = {n: t.float().clone() for n, t in a.iter_full_named_parameters()}
        b = make_engine(stage, fused=True, clip=clip)
        assert b.symm is not None, "peer-memory path did not come up"
        lb = run(b)
        b.symm.check()
        if clip == 0.0:  # without clipping the reduce-scatter feeds AdamW in the same kernel
            assert all(b._single_pass_update_ok(u) for u in b.units if u.grad_slot is None and u.checkpointed and u.n_train > 0)
            assert float(b.get_global_grad_norm()) == pytest_approx(float(a.get_global_grad_norm()))
        pb = {n: t.float().clone() for n, t in b.iter_full_named_parameters()}
        diff = max(float((pa[n] - pb[n]).abs().max()) for n in pa)
        res[f"stage{stage}_clip{clip}"] = {"nccl": la, "fused": lb, "max_param_diff": diff}
    if dist.get_rank() == 0:
        (Path(out_dir) / "fused_vs_nccl.json").write_text(json.dumps(res))


def scenario_copy_engine_gather(out_dir):
    """ZeRO-3 parameter gathers as peer copies on the copy engines against the pull kernel: the same bytes arrive, so
    losses and weights agree bit for bit."""
    os.environ["ATB200_GATHER"] = "kernel"
    a = make_engine(3, fused=True)
    assert not a._gather_on_copy_engines
    la = run(a)
    pa = {n: t.clone() for n, t in a.iter_full_named_parameters()}
    os.environ.pop("ATB200_GATHER")
    b = make_engine(3, fused=True)
    assert b._gather_on_copy_engines and b.symm is not None
    lb = run(b)
    b.symm.check()
    from arctictraining_b200.ops import COMM_COUNTER

    same = la == lb and all(torch.equal(pa[n], t) for n, t in b.iter_full_named_parameters())
    allsame = [None] * dist.get_world_size()
    dist.all_gather_object(allsame, bool(same))
    if dist.get_rank() == 0:
        (Path(out_dir) / "copy_engine_gather.json").write_text(json.dumps(
            {"same": all(allsame), "copies": int(COMM_COUNTER.get("copy_engine_all_gather", 0))}))


def scenario_nvls_reduce_scatter(out_dir):
    """Gradient reduce-scatter with the reduction done inside the NVSwitch (``multimem.ld_reduce`` on the multicast
    mapping of a symmetric buffer) against the peer-load kernel; reported as unavailable when the fabric offers no
    multicast mapping."""
    from arctictraining_b200.comm.symm import SymmetricContext

    rank, world = dist.get_rank(), dist.get_world_size()
    ctx = SymmetricContext(dist.group.WORLD, timeout_s=10.0)
    n = 8 * 4096
    buf = ctx.alloc("nvls_test", world * n, torch.bfloat16)
    res = {"multicast": bool(buf.multicast_ptr)}
    if buf.multicast_ptr:
        torch.manual_seed(rank)
        buf.tensor.copy_(torch.randn(world * n, device="cuda").bfloat16())
        ctx.barrier(slot=6)
        k = torch.ops.atb200
        a = torch.ones(n, device="cuda")
        sa = k.p2p_reduce_scatter_accum(buf.ptrs, rank * n, n, a, 0.5, False, True)
        b = torch.ones(n, device="cuda")
        sb = k.nvls_reduce_scatter_accum(buf.multicast_ptr, rank * n, n, b, 0.5, False, True)
        ctx.barrier(slot=6)
        ctx.check()
        # the switch adds the ranks' bf16 values in its own order and precision: equal up to bf16 rounding of the sum
        res["max_diff"] = float((a - b).abs().max())
        res["scale"] = float(a.abs().max())
        res["sumsq_rel"] = abs(float(sa) - float(sb)) / float(sa)
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        (Path(out_dir) / "nvls_reduce_scatter.json").write_text(json.dumps(allres))


def scenario_partly_frozen(out_dir):
    """Layers whose trainable prefix is shorter than one rank's shard (what LoRA or SwiftKV-style freezing produces):
    the ranks behind the frozen tail hold no trainable element of those units and must still take the same
    communication path as the others.  Also: two identical runs of the peer-memory path give bit-identical weights."""
    def build(fused, clip):
        e_cfg = load_arch_config("llama-3.1-8b", OVERRIDES)
        with torch.device("cuda"):
            m = CausalLM(e_cfg, dtype=torch.bfloat16)
        m.init_weights(seed=0)
        m.attn_impl = "sdpa"
        for layer in m.model.layers[1:]:
            for n, p in layer.named_parameters():
                p.requires_grad_("input_layernorm" in n)
        opt = FusedAdamW(OptimizerFactory.get_optimizer_grouped_params(m, 0.1), lr=1e-3, betas=(0.9, 0.95))
        return TrainingEngine(m, opt, None, {"zero_optimization": {"stage": 3}, "gradient_clipping": clip,
                                             "bfloat16": {"enabled": True}, "fused_comm": "auto" if fused else "off"})

    res = {}
    for clip in (1.0, 0.0):
        a = build(False, clip)
        la = run(a)
        pa = {n: t.float().clone() for n, t in a.iter_full_named_parameters()}
        runs = []
        for _ in range(2):
            b = build(True, clip)
            assert b.symm is not None, "peer-memory path did not come up"
            frozen_tail = [u for u in b.units if u.checkpointed and 0 < u.n_train < u.shard_size]
            assert frozen_tail, "the scenario needs units whose trainable prefix is shorter than a shard"
            assert all(b._fused_reduce_ok(u) for u in frozen_tail)
            lb = run(b)
            b.check_device_errors()
            runs.append((lb, {n: t.clone() for n, t in b.iter_full_named_parameters()}))
        diff = max(float((pa[n] - runs[0][1][n].float()).abs().max()) for n in pa)
        same = all(torch.equal(runs[0][1][n], runs[1][1][n]) for n in pa) and runs[0][0] == runs[1][0]
        res[f"clip{clip}"] = {"nccl": la, "fused": runs[0][0], "max_param_diff": diff, "bit_identical_reruns": bool(same),
                              "local_train_len": [u.train_len for u in frozen_tail]}
    allres = [None] * dist.get_world_size()
    dist.all_gather_object(allres, res)
    if dist.get_rank() == 0:
        (Path(out_dir) / "partly_frozen.json").write_text(json.dumps(allres))


def scenario_gather_gemm(out_dir):
    """ZeRO-3 gather inside the consuming GEMM: the weight that the staging CTAs assemble from the ranks' shards is
    bit-identical to what the pull all-gather assembles, and so is the product (odd sizes: a weight that starts in
    the middle of a shard, spans a shard boundary and ends in a partial tile)."""
    from arctictraining_b200.comm.symm import SymmetricContext
    from arctictraining_b200.ops import functional as Fn

    rank, P = dist.get_rank(), dist.get_world_size()
    ops = torch.ops.atb200
    symm = SymmetricContext(None)
    res = {}
    for name, (M, K, N, w_off, shard) in {
        "llama_qkv": (1024, 4096, 6144, 4096 * 8, ((4096 * 8 + 6144 * 4096 + 5000) // P + 255) // 256 * 256),
        "ragged": (300, 512, 1000, 1304, ((1304 + 1000 * 512 + 77) // P + 255) // 256 * 256),
    }.items():
        slab = symm.alloc(f"shards_{name}", shard, torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(7 + rank)
        slab.tensor.copy_((torch.randn(shard, device="cuda", generator=g) * 0.05).bfloat16())
        x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        full_a = torch.zeros(shard * P, device="cuda", dtype=torch.bfloat16)
        full_b = torch.zeros(shard * P, device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier()
        symm.all_gather(slab, 0, shard, full_a)
        ref = Fn.gemm(x, full_a[w_off : w_off + N * K].view(N, K))
        for _ in range(2):  # a second call reuses the arrival counters' allocation pattern
            full_b.zero_()
            got = ops.gemm_bf16_gather_b(x, slab.ptrs, 0, shard, full_b, w_off, N, 4)
        torch.cuda.synchronize()
        assert int(ops.read_and_clear_error_flag(x)) == 0
        symm.check()
        want = ref.float()
        res[name] = {
            "weight_equal": bool(torch.equal(full_b[w_off : w_off + N * K], full_a[w_off : w_off + N * K])),
            "outside_untouched": bool((full_b[:w_off] == 0).all() and (full_b[w_off + N * K :] == 0).all()),
            "out_equal": bool(torch.equal(got, ref)),
            "rel_err_vs_fp32": float((got.float() - x.float() @ full_a[w_off : w_off + N * K].view(N, K).float().t()).norm()
                                     / (want.norm() + 1e-12)),
        }
    allres = [None] * P
    dist.all_gather_object(allres, res)
    if rank == 0:
        (Path(out_dir) / "gather_gemm.json").write_text(json.dumps(allres))


def scenario_barrier_timeout(out_dir):
    """Rank 0 waits at a barrier that rank 1 joins only later: the wait runs out, the host sees an error status,
    and the context keeps working (plain peer loads, no multicast involved)."""
    from arctictraining_b200.comm.symm import SymmetricContext
    from arctictraining_b200.exceptions import CommTimeoutError

    ctx = SymmetricContext(None, timeout_s=0.5)
    rank = dist.get_rank()
    ok = True
    if rank == 0:
        ctx.barrier(slot=5)
        try:
            ctx.check()
            ok = False
        except CommTimeoutError:
            pass
        # the context is still usable
        t = torch.ones(4, device="cuda") * 3
        ok = ok and float(t.sum()) == 12.0
    dist.barrier()
    if rank != 0:
        ctx.barrier(slot=5)  # rank 0's flag is already there: returns at once
        ctx.check()
    ctx.timeout_s = 20.0
    ctx.barrier(slot=6)
    ctx.check()
    flags = [None] * dist.get_world_size()
    dist.all_gather_object(flags, ok)
    if rank == 0:
        (Path(out_dir) / "barrier_timeout.json").write_text(json.dumps({"ok": all(flags)}))


def scenario_ulysses_peer(out_dir):
    """The peer-memory Ulysses exchange gives the same attention output and input gradients as the NCCL one."""
    from types import SimpleNamespace

    from arctictraining_b200.parallel.ulysses import UlyssesContext

    rank, world = dist.get_rank(), dist.get_world_size()
    res = {}
    for name, (Hq, Hkv) in {"kv_split": (4, 2), "kv_replicated": (4, 1)}.items():
        torch.manual_seed(10 + rank)
        S_loc, D = 192, 128
        qkv = torch.randn(1, S_loc, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
        g = torch.randn(1, S_loc, Hq, D, device="cuda", dtype=torch.bfloat16)
        fctx = SimpleNamespace(cu_seqlens=None, max_seqlen=None, attn_impl="native")
        outs = []
        for fused in (False, True):
            sp = UlyssesContext(dist.group.WORLD, world, rank, fused=None if fused else False)
            x = qkv.clone().requires_grad_(True)
            q, k, v = x.view(1, S_loc, Hq + 2 * Hkv, D).split([Hq, Hkv, Hkv], dim=2)
            for _ in range(3):  # several exchanges in a row exercise the buffer rotation
                x.grad = None
                o = sp.attention(q, k, v, fctx)
                o.backward(g)
            assert fused is False or sp.fused is True, "peer exchange did not come up"
            if fused:
                sp._peer.symm.check()
            outs.append((o.detach().float(), x.grad.float()))
        # the exchange folded into the output projection GEMM, forward and backward
        w = (torch.randn(384, Hq * D, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)) * 0.05).bfloat16()
        resid = torch.randn(1, S_loc, 384, device="cuda", dtype=torch.bfloat16)
        gout = torch.randn(1, S_loc, 384, device="cuda", dtype=torch.bfloat16)
        got = []
        for use_fused in (True, False):
            x2 = qkv.clone().requires_grad_(True)
            w2 = w.clone().requires_grad_(True)
            r2 = resid.clone().requires_grad_(True)
            q2, k2, v2 = x2.view(1, S_loc, Hq + 2 * Hkv, D).split([Hq, Hkv, Hkv], dim=2)
            if use_fused:
                out = sp.attention_project(q2, k2, v2, fctx, w2, r2)
                assert out is not None, "fused projection path did not apply"
            else:
                out = r2 + torch.nn.functional.linear(sp.attention(q2, k2, v2, fctx).reshape(1, S_loc, Hq * D), w2)
            out.backward(gout)
            got.append([t.detach().float() for t in (out, x2.grad, w2.grad, r2.grad)])
        sp._peer.symm.check()
        assert int(torch.ops.atb200.read_and_clear_error_flag(w)) == 0
        proj_err = max(float((a - b).norm() / (b.norm() + 1e-12)) for a, b in zip(*got))
        res[name + "_proj_err"] = proj_err
        res[name] = {
            "out_diff": float((outs[0][0] - outs[1][0]).abs().max()),
            "grad_diff": float((outs[0][1] - outs[1][1]).abs().max()),
            "grad_scale": float(outs[0][1].abs().max()),
        }
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        (Path(out_dir) / "ulysses_peer.json").write_text(json.dumps(allres))


def scenario_fused_attention_block(out_dir):
    """A whole attention block under Ulysses: q|k|v projection pushing from its epilogue + rotary embedding after the
    exchange + gathering output projection, against projection / NCCL all-to-all / attention / projection."""
    from arctictraining_b200.models.arch import load_arch_config
    from arctictraining_b200.models.causal_lm import CausalLM
    from arctictraining_b200.parallel.ulysses import UlyssesContext

    rank, world = dist.get_rank(), dist.get_world_size()
    res = {}
    for name, (Hq, Hkv) in {"kv_split": (4, 2), "kv_replicated": (4, 1)}.items():
        cfg = load_arch_config("llama-3.1-8b", dict(num_hidden_layers=1, hidden_size=512, intermediate_size=1024,
                                                    num_attention_heads=Hq, num_key_value_heads=Hkv, vocab_size=1024,
                                                    head_dim=128))
        S_loc = 256
        got = []
        for fused in (True, False):
            with torch.device("cuda"):
                m = CausalLM(cfg, dtype=torch.bfloat16)
            m.init_weights(seed=0)
            m.attn_impl = "native"
            m.sp_context = UlyssesContext(dist.group.WORLD, world, rank, fused=None if fused else False)
            attn = m.model.layers[0].self_attn
            torch.manual_seed(7 + rank)
            x = torch.randn(1, S_loc, 512, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
            resid = torch.randn(1, S_loc, 512, device="cuda", dtype=torch.bfloat16)
            gout = torch.randn(1, S_loc, 512, device="cuda", dtype=torch.bfloat16)
            pos = (torch.arange(S_loc, device="cuda") + rank * S_loc)[None]
            ctx = m.build_context(pos)
            for _ in range(2):
                x.grad = None
                m.zero_grad()
                y = attn(x, ctx, residual=resid)
                y.backward(gout)
            if fused:
                assert "rope_global" in ctx.extras, "fused attention block was not taken"
                m.sp_context._peer.symm.check()
            assert int(torch.ops.atb200.read_and_clear_error_flag(x)) == 0
            got.append([t.detach().float() for t in (y, x.grad, attn.qkv_proj.weight.grad, attn.o_proj.weight.grad)])
        res[name] = max(float((a - b).norm() / (b.norm() + 1e-12)) for a, b in zip(*got))
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        (Path(out_dir) / "fused_attention_block.json").write_text(json.dumps(allres))


def scenario_moe_peer(out_dir):
    """Expert-parallel MoE block: the peer-memory dispatch/combine gives the same output and gradients as the NCCL
    all-to-all path."""
    from arctictraining_b200.moe.layer import ArcticMoE
    from arctictraining_b200.moe.layer import MoEConfig

    rank, world = dist.get_rank(), dist.get_world_size()
    res = {}
    outs = []
    for fused in (False, True):
        os.environ["ATB200_FUSED_COMM"] = "1" if fused else "0"
        import arctictraining_b200.moe.peer as peer

        peer._EXCHANGES.clear()
        torch.manual_seed(0)
        mc = MoEConfig(model_dim=256, intermediate_dim=128, num_experts=8, top_k=2, normalize_topk_scores=True,
                       loss_coeff=0.0, ep_size=world, ep_rank=rank, ep_group=dist.group.WORLD, input_dtype=torch.bfloat16)
        moe = ArcticMoE(mc, dtype=torch.bfloat16, device="cuda")
        g = torch.Generator(device="cuda").manual_seed(5)
        for n, p in sorted(moe.named_parameters()):
            full = torch.randn(p.shape if "expert" not in n else (8,) + tuple(p.shape[1:]), generator=g, device="cuda") * 0.05
            p.data.copy_((full[rank * 4 : rank * 4 + 4] if "expert" in n else full).to(p.dtype))
        torch.manual_seed(100 + rank)
        x = torch.randn(1, 333, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        gy = torch.randn(1, 333, 256, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            x.grad = None
            moe.zero_grad()
            y = moe(x)
            y.backward(gy)
        if fused:
            assert peer.exchange_for(dist.group.WORLD) is not None, "peer exchange did not come up"
            peer.check_errors()
        outs.append((y.detach().float(), x.grad.float(), moe.expert_down.grad.float(), moe.router_gate.grad.float()))

    def rel(a, b):
        return float((a - b).norm() / (b.norm() + 1e-12))

    res = {k: rel(outs[1][i], outs[0][i]) for i, k in enumerate(["out", "dx", "dw_down", "d_router"])}
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        (Path(out_dir) / "moe_peer.json").write_text(json.dumps(allres))


def scenario_embed_gather(out_dir):
    """Peer-memory gather of query | document embeddings against the NCCL gather: same values, twice in a row (both
    halves of the rotating buffer), and the local rows carry gradients."""
    from arctictraining_b200.comm.symm import SymmetricContext
    from arctictraining_b200.embed.trainer import PeerEmbeddingGather
    from arctictraining_b200.embed.trainer import gather_embeddings

    rank, world = dist.get_rank(), dist.get_world_size()
    gather = PeerEmbeddingGather(SymmetricContext(dist.group.WORLD, timeout_s=10.0))
    ok = True
    for step in range(3):
        torch.manual_seed(100 * step + rank)
        q = torch.randn(6, 72, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        d = torch.randn(13, 72, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        fq, fd = gather(q, d, rank, world)
        rq, rd = gather_embeddings(q, rank, world), gather_embeddings(d, rank, world)
        ok &= torch.equal(fq, rq) and torch.equal(fd, rd)
        (fq.float().sum() * 2 + fd.float().sum() * 3).backward()
        ok &= bool((q.grad == 2).all()) and bool((d.grad == 3).all())
    gather.symm.check()
    allok = [None] * world
    dist.all_gather_object(allok, bool(ok))
    if rank == 0:
        (Path(out_dir) / "embed_gather.json").write_text(json.dumps({"ok": all(allok)}))


def main():
    scenario, out_dir = sys.argv[1], sys.argv[2]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch._C._set_print_stack_traces_on_fatal_signal(True)  # a crash in native code reports where
    init_distributed(timeout_s=120)
    {"fused_vs_nccl": scenario_fused_vs_nccl, "barrier_timeout": scenario_barrier_timeout, "partly_frozen": scenario_partly_frozen, "gather_gemm": scenario_gather_gemm,
     "ulysses_peer": scenario_ulysses_peer, "moe_peer": scenario_moe_peer,
     "fused_attention_block": scenario_fused_attention_block, "embed_gather": scenario_embed_gather,
     "copy_engine_gather": scenario_copy_engine_gather, "nvls_reduce_scatter": scenario_nvls_reduce_scatter}[scenario](out_dir)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.argv = [a for a in sys.argv if not a.startswith("--local_rank")]
    main()
