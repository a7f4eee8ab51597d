# SPDX-License-Identifier: Apache-2.0
"""Data-movement kernels of csrc/comm_p2p.cu on ONE GPU: the "peers" are separate local buffers, every
emulated rank is launched in turn (none of these kernels waits on another rank)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k():
    from arctictraining_b200.ops import _ext

    _ext.require()
    return torch.ops.atb200


def ptrs(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64)


def test_all_gather_pull(k):
    P, n = 4, 4096 + 64
    shards = [torch.randn(n + 16, device="cuda").bfloat16() for _ in range(P)]
    full = torch.empty(P * n, device="cuda", dtype=torch.bfloat16)
    k.p2p_all_gather(ptrs(shards), 16 * 2, full, n, 0)
    assert torch.equal(full, torch.cat([s[16 : 16 + n] for s in shards]))


def test_reduce_scatter_accumulate_and_norm(k):
    torch.manual_seed(0)
    P, total = 4, 8 * 4096
    grads = [torch.randn(total, device="cuda").bfloat16() for _ in range(P)]
    n = total // P
    for r in range(P):
        acc = torch.ones(n, device="cuda")
        ss = k.p2p_reduce_scatter_accum(ptrs(grads), r * n, n, acc, 0.25, False, True)
        ref = 1 + 0.25 * sum(g[r * n : (r + 1) * n].float() for g in grads)
        assert torch.allclose(acc, ref, atol=1e-5)
        assert abs(float(ss) - float(ref.pow(2).sum())) / float(ref.pow(2).sum()) < 1e-5
        acc2 = torch.full((n,), 7.0, device="cuda")
        k.p2p_reduce_scatter_accum(ptrs(grads), r * n, n, acc2, 1.0, True, False)
        assert torch.allclose(acc2, ref * 4 - 4, atol=1e-4)


def test_reduce_scatter_adamw_matches_two_pass(k):
    torch.manual_seed(0)
    P, n = 2, 8 * 1024
    grads = [torch.randn(2 * n, device="cuda").bfloat16() for _ in range(P)]
    master = torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref_p, ref_m, ref_v = master.clone(), m.clone(), v.clone()
    g = 0.5 * sum(x[n : 2 * n].float() for x in grads)
    k.adamw_step(ref_p, g, ref_m, ref_v, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, None)
    ss = k.p2p_reduce_scatter_adamw(ptrs(grads), n, n, 0.5, master, m, v, lp, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1)
    assert torch.allclose(master, ref_p, atol=1e-6) and torch.allclose(m, ref_m, atol=1e-7) and torch.allclose(v, ref_v, atol=1e-7)
    assert torch.allclose(lp.float(), master, atol=2e-2)
    assert abs(float(ss) - float(g.pow(2).sum())) / float(g.pow(2).sum()) < 1e-5


def test_ulysses_exchanges_are_inverse_and_match_reference(k):
    torch.manual_seed(0)
    P, S_loc, H, D = 4, 37, 8, 64
    xs = [torch.randn(S_loc, H, D, device="cuda").bfloat16() for _ in range(P)]
    ys = [torch.empty(P * S_loc, H // P, D, device="cuda", dtype=torch.bfloat16) for _ in range(P)]
    for r in range(P):
        k.p2p_seq_to_head(xs[r], ptrs(ys), r, False)
    full = torch.cat(xs, dim=0)  # [S, H, D]
    for o in range(P):
        assert torch.equal(ys[o], full[:, o * (H // P) : (o + 1) * (H // P)])
    back = [torch.empty(S_loc, H, D, device="cuda", dtype=torch.bfloat16) for _ in range(P)]
    for r in range(P):
        k.p2p_seq_to_head(ys[r], ptrs(back), r, True)
    for r in range(P):
        assert torch.equal(back[r], xs[r])


def test_moe_dispatch_and_combine_through_peer_buffers(k):
    torch.manual_seed(0)
    P, E, K, T, H = 2, 8, 2, 300, 64
    El = E // P
    experts = [torch.randint(0, E, (T, K), device="cuda", dtype=torch.int32) for _ in range(P)]
    xs = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(P)]
    local = [k.moe_assign_slots(e, E, 1) for e in experts]  # (slots, counts, offsets)
    all_counts = torch.stack([l[1] for l in local]).contiguous()
    rows = P * T * K + El * 127
    bufs = [torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16) for _ in range(P)]
    dests, segs = [], []
    for r in range(P):
        d, seg = k.moe_dest_rows(all_counts, experts[r], local[r][0], local[r][2], r, 128)
        dests.append(d)
        segs.append(seg)
        k.p2p_moe_dispatch(xs[r], experts[r], d, ptrs(bufs), 0, El, rows, None)
    torch.cuda.synchronize()
    # owner-side check: segment of local expert e on rank o holds the rows of rank 0 first, then rank 1, in (token, k) order
    for o in range(P):
        seg = segs[o].tolist()
        assert all(s % 128 == 0 for s in seg)
        for el in range(El):
            e = o * El + el
            want = torch.cat([xs[r][(experts[r] == e).nonzero()[:, 0]] for r in range(P)])
            got = bufs[o][seg[el] : seg[el] + want.shape[0]]
            assert torch.equal(got, want), (o, el)
    scores = [torch.rand(T, K, device="cuda") for _ in range(P)]
    for r in range(P):
        out = k.p2p_moe_combine(ptrs(bufs), 0, experts[r], dests[r], scores[r], H, El, rows)
        ref = xs[r].float() * scores[r].sum(-1, keepdim=True)
        assert (out.float() - ref).norm() / ref.norm() < 1e-2
        # gradient of the combine weights: <dout[t], y[pair]> with y = the dispatched copy of x[t]
        dout = torch.randn(T, H, device="cuda").bfloat16()
        dots = k.p2p_moe_pair_dot(ptrs(bufs), 0, experts[r], dests[r], dout, El, rows)
        want = (dout.float() * xs[r].float()).sum(-1, keepdim=True).expand(T, K)
        assert torch.allclose(dots, want, atol=1e-2, rtol=1e-3)
    # scaled dispatch (backward of the combine) and the capacity guard
    k.comm_read_and_clear_error(xs[0])
    k.p2p_moe_dispatch(xs[0], experts[0], dests[0], ptrs(bufs), 0, El, rows, scores[0])
    assert int(k.comm_read_and_clear_error(xs[0])) == 0
    k.p2p_moe_dispatch(xs[0], experts[0], dests[0], ptrs(bufs), 0, El, 8, None)  # capacity far too small: rows are skipped
    assert int(k.comm_read_and_clear_error(xs[0])) >> 8 == 0x31


def test_reduce_scatter_is_bit_identical_on_a_second_run_and_writes_only_its_slice(k):
    """The reduction adds the peers' pieces in rank order, so two runs give the same bits; the accumulator lives inside a
    larger buffer filled with a canary value, which must survive around the written slice (odd length: tail path)."""
    torch.manual_seed(1)
    P, n, pad = 4, 8 * 1000 + 8, 64
    grads = [torch.randn(P * n, device="cuda").bfloat16() for _ in range(P)]
    outs = []
    for _ in range(2):
        buf = torch.full((n + 2 * pad,), -123.25, device="cuda")
        acc = buf[pad : pad + n]
        ss = k.p2p_reduce_scatter_accum(ptrs(grads), 2 * n, n, acc, 0.5, True, True)
        outs.append((acc.clone(), ss.clone()))
        assert bool((buf[:pad] == -123.25).all()) and bool((buf[pad + n :] == -123.25).all())
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_all_gather_writes_only_the_requested_range(k):
    P, n, pad = 3, 8 * 500, 32
    shards = [torch.randn(n, device="cuda").bfloat16() for _ in range(P)]
    buf = torch.full((P * n + 2 * pad,), 7.5, device="cuda", dtype=torch.bfloat16)
    k.p2p_all_gather(ptrs(shards), 0, buf[pad : pad + P * n], n, 0)
    assert torch.equal(buf[pad : pad + P * n], torch.cat(shards))
    assert bool((buf[:pad] == 7.5).all()) and bool((buf[pad + P * n :] == 7.5).all())
