"""Peer-memory communication kernels, with several ranks emulated inside one GPU.

The kernels of all pretend ranks run one after another on one device: first every rank's send kernel,
then every rank's wait kernel, so no kernel ever waits for work that has not been launched yet.  The
"peers" are separate buffers on the same GPU, addressed through the same pointer tables a real
multi-GPU run uses.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def cops():
    from moe_distributed_training_b200.ops import cuda_ops
    return cuda_ops


@pytest.mark.parametrize("ws,E,k,tokens", [(2, 4, 2, [300, 77]), (4, 8, 2, [513, 128, 1000, 5]), (1, 4, 2, [200])])
def test_dispatch_and_combine_emulated_ranks(cops, ws, E, k, tokens):
    from moe_distributed_training_b200.parallel import symm
    ext = cops.ext
    H, El = 256, E // ws
    torch.manual_seed(0)
    spaces = symm.emulate_ep_workspaces(ws, E, H, max(tokens), k, DEV)
    status = cops.status_tensor(DEV)
    xs = [torch.randn(t, H, device=DEV).to(torch.bfloat16) for t in tokens]
    tops = [torch.randn(t, E, device=DEV).topk(k, -1).indices.int() for t in tokens]
    plans = [cops.make_plan(tp, E, 1, tp.numel()) for tp in tops]
    off = [int(v) for v in ext.ep_meta_offsets(ws, E)]
    metas = [torch.zeros(off[8], dtype=torch.int32, device=DEV) for _ in range(ws)]
    for epoch in (1, 2):      # two exchanges in a row: parities alternate, counters are re-used
        par = epoch & 1
        for r, w in enumerate(spaces):
            ext.ep_counts_send(plans[r].tokens_per_expert, w.peer_base, w.layout, r, par, epoch)
        for r, w in enumerate(spaces):
            ext.ep_counts_wait_meta(w.my_base, w.layout, r, par, epoch, metas[r], status)
        for r, w in enumerate(spaces):
            ext.ep_dispatch(xs[r], plans[r].src_slot, tops[r].reshape(-1).contiguous(), None, metas[r], w.peer_base, w.layout, r, k, par, status)
        for r, w in enumerate(spaces):
            ext.ep_recv_prepare(w.my_base, w.layout, metas[r], H, par, status, True)
        cops.check_status(DEV)
        # oracle of every receive buffer
        for d, w in enumerate(spaces):
            rows = []
            for le in range(El):
                e = d * El + le
                seg = []
                for s in range(ws):
                    flat = tops[s].reshape(-1)
                    slots = (flat == e).nonzero().flatten()          # stable slot order
                    seg.append(xs[s][slots // k])
                seg = torch.cat(seg)
                pad = (-seg.shape[0]) % 128
                rows.append(torch.cat([seg, torch.zeros(pad, H, device=DEV, dtype=torch.bfloat16)]))
            want = torch.cat(rows)
            m = metas[d].cpu()
            assert int(m[off[7] + 2]) == want.shape[0]
            assert torch.equal(w.recv_x()[:want.shape[0]], want), f"rank {d} receive buffer"
        # combine: send 2x the received rows back
        ys = [w.recv_x() * 2 for w in spaces]
        for r, w in enumerate(spaces):
            ext.ep_combine_send(ys[r], metas[r], w.peer_base, w.layout, r, w.capacity_rows, par, status)
        for r, w in enumerate(spaces):
            ext.ep_wait_rows(w.my_base, w.layout, metas[r], par, status, 1)
        cops.check_status(DEV)
        for r, w in enumerate(spaces):
            n = tops[r].numel()
            want = 2 * xs[r][(plans[r].src_slot[:n] // k).long()]
            assert torch.equal(w.recv_y()[:n], want), f"rank {r} returned rows"


def test_flat_all_gather_and_reduce_scatter_emulated(cops):
    ext = cops.ext
    ws, n = 4, 4096 + 512
    torch.manual_seed(1)
    shards = [torch.randn(n, device=DEV).to(torch.bfloat16) for _ in range(ws)]
    table = torch.tensor([s.data_ptr() for s in shards], dtype=torch.int64, device=DEV)
    out = torch.empty(ws * n, dtype=torch.bfloat16, device=DEV)
    ext.ag_pull(out, table, ws, 0, n * 2)
    assert torch.equal(out, torch.cat(shards))
    fulls = [torch.randn(ws * n, device=DEV) for _ in range(ws)]
    ftable = torch.tensor([f.data_ptr() for f in fulls], dtype=torch.int64, device=DEV)
    for rank in range(ws):
        acc = torch.ones(n, dtype=torch.bfloat16, device=DEV)
        ext.rs_pull(acc, ftable, ws, rank, True, 0.25, True)
        want = 1.0 + 0.25 * sum(f[rank * n:(rank + 1) * n] for f in fulls)
        assert torch.allclose(acc.float(), want, atol=2e-2, rtol=2e-2)


def test_peer_wait_gives_up_with_a_status_code(cops):
    """A flag that nothing sets: the wait runs out after its (here 200 ms) limit, the kernel returns and
    reports code 5 in the status word; the context stays usable."""
    ext = cops.ext
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ext.barrier_wait(flags.data_ptr(), 2, 1, status, 200)
    torch.cuda.synchronize()
    assert int(status.item()) == 5
    flags.fill_(1)
    status.zero_()
    ext.barrier_wait(flags.data_ptr(), 2, 1, status, 200)
    torch.cuda.synchronize()
    assert int(status.item()) == 0


@pytest.fixture(params=[0, 4], ids=["tile128", "tall"])
def gemm_tile_policy(request, cops):
    """Runs a test with the 128-row GEMM kernel and with the tall 256 x 256 kernel forced."""
    prev = cops.ext.gemm_set_pair_policy(request.param)
    yield request.param
    cops.ext.gemm_set_pair_policy(prev)


@pytest.mark.parametrize("ws,E,tokens", [(2, 4, [300, 77]), (4, 8, [513, 128, 700, 5])])
def test_gemm_takes_part_in_the_exchange_emulated_ranks(cops, ws, E, tokens, gemm_tile_policy):
    """Grouped GEMM that waits for its row tiles on the arrival counters and stores its result rows straight
    into the source ranks' buffers, for several ranks emulated on one GPU (all sends before any GEMM)."""
    from moe_distributed_training_b200.ops.reference import RoutingPlan
    from moe_distributed_training_b200.parallel import symm
    ext = cops.ext
    H, N, k, El = 256, 512, 2, E // ws
    torch.manual_seed(3)
    spaces = symm.emulate_ep_workspaces(ws, E, N, max(tokens), k, DEV)   # recv rows have N columns on the way back
    # the forward buffer holds H-column rows: use a second set of workspaces for the inputs
    spaces_in = symm.emulate_ep_workspaces(ws, E, H, max(tokens), k, DEV)
    status = cops.status_tensor(DEV)
    W = (torch.randn(E, N, H, device=DEV) * 0.05).to(torch.bfloat16)
    xs = [torch.randn(t, H, device=DEV).to(torch.bfloat16) for t in tokens]
    tops = [torch.randn(t, E, device=DEV).topk(k, -1).indices.int() for t in tokens]
    plans = [cops.make_plan(tp, E, 1, tp.numel()) for tp in tops]
    off = [int(v) for v in ext.ep_meta_offsets(ws, E)]
    metas = [torch.zeros(off[8], dtype=torch.int32, device=DEV) for _ in range(ws)]
    for epoch in (1, 2):
        par = epoch & 1
        for r, w in enumerate(spaces_in):
            ext.ep_counts_send(plans[r].tokens_per_expert, w.peer_base, w.layout, r, par, epoch)
        for r, w in enumerate(spaces_in):
            ext.ep_counts_wait_meta(w.my_base, w.layout, r, par, epoch, metas[r], status)
        for r, w in enumerate(spaces_in):
            ext.ep_dispatch(xs[r], plans[r].src_slot, tops[r].reshape(-1).contiguous(), None, metas[r], w.peer_base, w.layout, r, k, par, status)
        for r, w in enumerate(spaces_in):
            ext.ep_recv_prepare(w.my_base, w.layout, metas[r], H, par, status, False)
        for r, (wi, wo) in enumerate(zip(spaces_in, spaces)):
            rr, rp, te = ext.ep_fused_meta(metas[r], wi.layout, r)
            m = metas[r]
            rplan = RoutingPlan(m[off[1]:off[1] + El], m[off[2]:off[2] + El + 1], None, None, 1, El, capacity_rows=wi.capacity_rows)
            peer_out = torch.tensor([b + wo.layout[9] for b in wo.bases], dtype=torch.int64, device=DEV)
            peer_arr = torch.tensor([b + wo.layout[7] + 4 * par for b in wo.bases], dtype=torch.int64, device=DEV)
            dummy = torch.empty(wi.capacity_rows, N, dtype=torch.bfloat16, device=DEV)
            cops._g(1, wi.recv_x(), False, W[r * El:(r + 1) * El], False, dummy, N, H, rplan,
                    wait=(wi.tile_counters(par), te), scatter=(rr, rp, peer_out, peer_arr))
        for r, wo in enumerate(spaces):
            ext.ep_wait_rows(wo.my_base, wo.layout, metas[r], par, status, (N + 255) // 256)
        cops.check_status(DEV)
        for r, wo in enumerate(spaces):
            n = tops[r].numel()
            slot = plans[r].src_slot[:n].long()
            e = tops[r].reshape(-1)[slot].long()
            want = torch.einsum("nh,nkh->nk", xs[r][slot // k].float(), W[e].float())
            got = wo.recv_y()[:n].float()
            err = (got - want).norm() / want.norm()
            assert err < 2e-2, (r, float(err))


def test_exchange_is_inert_after_a_counts_wait_that_ran_out(cops):
    """A peer whose counts never arrive: the counts wait gives up after its (here 100 ms) limit, reports code 5 and
    writes metadata that describe no rows.  Every later kernel of the exchange, the GEMM that takes part in it
    included, must then leave all workspaces exactly as they were."""
    from moe_distributed_training_b200.ops.reference import RoutingPlan
    from moe_distributed_training_b200.parallel import symm
    ext = cops.ext
    ws, E, k, H, N, T = 2, 4, 2, 256, 256, 300
    El = E // ws
    torch.manual_seed(5)
    spaces = symm.emulate_ep_workspaces(ws, E, H, T, k, DEV)
    status = cops.status_tensor(DEV)
    status.zero_()
    x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    top = torch.randn(T, E, device=DEV).topk(k, -1).indices.int()
    plan = cops.make_plan(top, E, 1, top.numel())
    off = [int(v) for v in ext.ep_meta_offsets(ws, E)]
    meta = torch.full((off[8],), 12345, dtype=torch.int32, device=DEV)     # stands for uninitialised memory
    W = (torch.randn(El, N, H, device=DEV) * 0.05).to(torch.bfloat16)
    w = spaces[0]
    ext.set_peer_wait_limit_ms(100)
    try:
        ext.ep_counts_send(plan.tokens_per_expert, w.peer_base, w.layout, 0, 1, 1)     # rank 1 never sends its counts
        torch.cuda.synchronize()
        before = [sp.buffer.clone() for sp in spaces]
        ext.ep_counts_wait_meta(w.my_base, w.layout, 0, 1, 1, meta, status)
        ext.ep_dispatch(x, plan.src_slot, top.reshape(-1).contiguous(), None, meta, w.peer_base, w.layout, 0, k, 1, status)
        ext.ep_recv_prepare(w.my_base, w.layout, meta, H, 1, status, False)
        rr, rp, te = ext.ep_fused_meta(meta, w.layout, 0)
        rplan = RoutingPlan(meta[off[1]:off[1] + El], meta[off[2]:off[2] + El + 1], None, None, 1, El, capacity_rows=w.capacity_rows)
        peer_out = torch.tensor([b + w.layout[9] for b in w.bases], dtype=torch.int64, device=DEV)
        peer_arr = torch.tensor([b + w.layout[7] + 4 for b in w.bases], dtype=torch.int64, device=DEV)
        dummy = torch.empty(w.capacity_rows, N, dtype=torch.bfloat16, device=DEV)
        cops._g(1, w.recv_x(), False, W, False, dummy, N, H, rplan, wait=(w.tile_counters(1), te), scatter=(rr, rp, peer_out, peer_arr))
        ext.ep_combine_send(w.recv_x(), meta, w.peer_base, w.layout, 0, w.capacity_rows, 1, status)
        ext.ep_wait_rows(w.my_base, w.layout, meta, 1, status, 1)
        torch.cuda.synchronize()
        assert int(status.item()) == 5
        assert int(meta.abs().sum()) == 0, "metadata of a failed exchange must describe no rows"
        for sp, b in zip(spaces, before):
            assert torch.equal(sp.buffer, b), "a kernel of the failed exchange wrote into a workspace"
    finally:
        ext.set_peer_wait_limit_ms(0)
        status.zero_()


def test_flagged_all_gather_feeds_a_gemm_chunk_by_chunk(cops):
    """All-gather with progress flags on a side stream; the GEMM on the main stream finds its weight operand in the
    registry of gathered buffers and waits for the chunks each output tile needs.  Two rounds into the same buffer
    (the second with new weights and the next epoch) and both operand layouts (x W^T per row panel, dy W whole)."""
    ext = cops.ext
    ws, N, K, M = 4, 1536, 1024, 300
    torch.manual_seed(7)
    status = cops.status_tensor(DEV)
    n_el = N * K
    assert n_el % (ws * 128) == 0
    shard = n_el // ws
    nflags, chunk_bytes = ext.ag_chunks(ws, shard * 2)
    ready = torch.zeros(nflags, dtype=torch.int32, device=DEV)
    out = torch.zeros(n_el, dtype=torch.bfloat16, device=DEV)
    side = torch.cuda.Stream()
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    dy = torch.randn(M, N, device=DEV).to(torch.bfloat16)
    ext.set_peer_wait_limit_ms(2000)
    try:
        for epoch in (1, 2):
            Wfull = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
            shards = [Wfull.reshape(-1)[r * shard:(r + 1) * shard].clone() for r in range(ws)]
            table = torch.tensor([s_.data_ptr() for s_ in shards], dtype=torch.int64, device=DEV)
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                ext.ag_pull_flagged(out, table, ws, 1, shard * 2, ready, epoch, 1)
            W = out.view(N, K)
            y = cops.mm_nt(x, W)            # rows n0 .. n0+255 of W per output tile
            dx = cops.mm_nn(dy, W)          # the whole of W for every tile
            torch.cuda.synchronize()
            cops.check_status(DEV)
            assert torch.equal(out, Wfull.reshape(-1))
            assert int(ready.min()) == epoch and int(ready.max()) == epoch
            for got, want in ((y, x.float() @ Wfull.float().t()), (dx, dy.float() @ Wfull.float())):
                err = (got.float() - want).norm() / want.norm()
                assert err < 1e-2, float(err)
    finally:
        ext.set_peer_wait_limit_ms(0)
        ext.gather_registry_clear()


def test_reduce_scatter_block_kernel_emulated(cops):
    """announce + wait + reduce in one kernel.  With the ranks emulated on one GPU their kernels run one after another,
    so the peers' announcements are written by the test beforehand; a second case leaves them out and lets the
    (100 ms) wait run out: status 5, output untouched."""
    ext = cops.ext
    ws, n = 4, 4096 + 512 + 4
    torch.manual_seed(11)
    fulls = [torch.randn(ws * n, device=DEV) for _ in range(ws)]
    ftable = torch.tensor([f.data_ptr() for f in fulls], dtype=torch.int64, device=DEV)
    flags = [torch.zeros(8 * ws, dtype=torch.int32, device=DEV) for _ in range(ws)]
    flag_table = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for f in flags:
        f.view(8, ws)[3].fill_(7)          # slot 3, epoch 7: every rank has announced
    for rank in range(ws):
        acc = torch.ones(n, dtype=torch.bfloat16, device=DEV)
        ext.rs_block(acc, ftable, flag_table, flags[rank].data_ptr(), 3, ws, rank, True, 0.25, True, 7, status)
        want = 1.0 + 0.25 * sum(f[rank * n:(rank + 1) * n] for f in fulls)
        assert torch.allclose(acc.float(), want, atol=2e-2, rtol=2e-2)
    assert int(status.item()) == 0
    # the all-reduce form: every rank gets the sum of the whole buffers (bf16 in, bf16 out)
    parts = [torch.randn(n, device=DEV).to(torch.bfloat16) for _ in range(ws)]
    ptable = torch.tensor([p_.data_ptr() for p_ in parts], dtype=torch.int64, device=DEV)
    for f in flags:
        f.view(8, ws)[5].fill_(2)
    for rank in range(ws):
        out = torch.empty(n, dtype=torch.bfloat16, device=DEV)
        ext.rs_block(out, ptable, flag_table, flags[rank].data_ptr(), 5, ws, rank, False, 1.0, False, 2, status, 0, True)
        assert torch.allclose(out.float(), sum(p_.float() for p_ in parts), atol=3e-2, rtol=2e-2)
    assert int(status.item()) == 0
    ext.set_peer_wait_limit_ms(100)
    try:
        acc = torch.ones(n, dtype=torch.bfloat16, device=DEV)
        ext.rs_block(acc, ftable, flag_table, flags[0].data_ptr(), 4, ws, 0, True, 0.25, True, 9, status)   # nobody else announces
        torch.cuda.synchronize()
        assert int(status.item()) == 5
        assert torch.equal(acc, torch.ones_like(acc))
    finally:
        ext.set_peer_wait_limit_ms(0)
