"""Peer-memory exchange of partials fused with the combine (tk_peer_*), on one GPU: the ranks live
in this process, are connected with their mailbox addresses, and are driven the only way ranks that
share a GPU may be driven - every send before any receive, so that no kernel waits for a later
launch.  The fused single-kernel form runs across real GPUs in tests/test_gpu_multi.py."""
import numpy as np
import pytest
import torch

from titan_engine_b200 import dist as D

pytestmark = pytest.mark.gpu


def _partials(gen, n_rows, dv, dev):
    p = torch.randn(n_rows, dv + 2, device=dev, generator=gen)
    p[:, dv] = torch.randn(n_rows, device=dev, generator=gen) * 3.0            # running maxima
    p[:, dv + 1] = torch.rand(n_rows, device=dev, generator=gen) * 50.0 + 0.1  # sums of weights
    return p.contiguous()


@pytest.mark.parametrize("world,n_rows,dv", [(3, 32, 128), (2, 1, 64), (8, 257, 128)])
def test_send_then_recv_combine_equals_combine_of_stack(world, n_rows, dv):
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev); gen.manual_seed(100 + world)
    ranks = [D.PeerExchange(n_rows + 3, dv + 2, rank=r, world=world, connect=False) for r in range(world)]
    for r in ranks:
        r.connect_local(ranks)
    for epoch in range(5):                                  # both parities, reused
        n = n_rows if epoch != 2 else max(1, n_rows // 2)   # fewer rows than the mailbox holds
        parts = [_partials(gen, n, dv, dev) for _ in range(world)]
        for r, p in zip(ranks, parts):
            r.send(p)
        want = D.combine_partials(torch.stack(parts).view(world, 1, n, dv + 2), torch.float32).view(n, dv)
        for r, p in zip(ranks, parts):
            got = r.recv_combine(p, torch.float32)
            r.status()
            assert torch.equal(got, want), f"epoch {epoch} rank {r.rank}: max diff {(got - want).abs().max().item()}"
        got16 = ranks[0].recv_combine(parts[0], torch.bfloat16)
        assert torch.equal(got16, want.to(torch.bfloat16))
    for r in ranks:
        r.close()


def test_world_of_one_is_a_plain_combine():
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev); gen.manual_seed(7)
    ex = D.PeerExchange(16, 130, rank=0, world=1)
    p = _partials(gen, 16, 128, dev)
    got = ex.exchange_combine(p, torch.float32)
    want = D.combine_partials(p.view(1, 1, 16, 130), torch.float32).view(16, 128)
    ex.status()
    assert torch.equal(got, want)
    ex.close()


def test_missing_peer_runs_into_the_wait_limit_and_reports_timeout():
    """Rank 1 never sends: rank 0's wait gives up after its limit, the status says so, the output is
    left alone and the context stays usable (a later complete exchange works)."""
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev); gen.manual_seed(8)
    ranks = [D.PeerExchange(8, 130, rank=r, world=2, connect=False) for r in range(2)]
    for r in ranks:
        r.connect_local(ranks)
        r.set_wait_limit_ms(50)
    p0, p1 = _partials(gen, 8, 128, dev), _partials(gen, 8, 128, dev)
    ranks[0].exchange_combine(p0, torch.float32)            # sends, then waits for rank 1 in vain
    with pytest.raises(RuntimeError, match="status 4"):
        ranks[0].status()
    ranks[0].status()                                       # the flag is cleared by the read
    # rank 1 catches up with the epoch rank 0 is in; then a complete round
    ranks[1].send(p1)
    got = ranks[0].recv_combine(p0, torch.float32)
    ranks[0].status()
    want = D.combine_partials(torch.stack([p0, p1]).view(2, 1, 8, 130), torch.float32).view(8, 128)
    assert torch.equal(got, want)
    assert float(torch.ones(4, device=dev).sum()) == 4.0
    for r in ranks:
        r.close()


def test_argument_checks():
    ex = D.PeerExchange(4, 130, rank=0, world=2, connect=False)
    p = torch.zeros(4, 130, device="cuda")
    with pytest.raises(RuntimeError, match="not connected"):
        ex.send(p)
    ex.connect_local([ex, ex])
    with pytest.raises(RuntimeError, match="do not fit"):
        ex.send(torch.zeros(5, 130, device="cuda"))
    with pytest.raises(AssertionError):
        ex.send(torch.zeros(4, 66, device="cuda"))
    ex.close()
    with pytest.raises(RuntimeError):
        D.PeerExchange(4, 131, rank=0, world=1)             # odd row width
    with pytest.raises(RuntimeError):
        D.PeerExchange(4, 130, rank=0, world=17)


def _split_caches(dev, n, H, Hkv, D, world, gen):
    """One sequence of n tokens: `whole` holds all of it, parts[r] holds rank r's page-aligned range."""
    from titan_engine_b200 import PagedKVCache
    pg = n // 16
    full = torch.randn(pg, Hkv, 2, 16, D, device=dev, generator=gen).to(torch.bfloat16)
    whole = PagedKVCache(1, H, Hkv, D, pg, 1, pg, dtype="bf16")
    ws = whole.seq_alloc(); whole.adopt(ws, np.arange(pg, dtype=np.int32), n)
    whole.layer_views(0)[0].copy_(full)
    whole.step_begin([ws], None)
    parts = []
    for lo, hi in D_ranges(n, world):
        mp = (hi - lo) // 16
        c = PagedKVCache(1, H, Hkv, D, mp, 1, mp, dtype="bf16")
        s = c.seq_alloc(); c.adopt(s, np.arange(mp, dtype=np.int32), hi - lo)
        c.layer_views(0)[0].copy_(full[lo // 16:hi // 16])
        c.step_begin([s], None)
        parts.append(c)
    return whole, parts


def D_ranges(n, world):
    return D.token_ranges(n, world)


@pytest.mark.parametrize("shape", [(32, 8, 128), (8, 8, 64), (16, 1, 128)])
def test_attention_kernel_carries_the_exchange_and_meets_the_two_launch_route(shape):
    """Two ranks in this process, each with half of one sequence.  The rank that goes second runs
    tk_kv_decode_exchange as ONE launch (its merging CTAs find the first rank's rows already
    there); the rank that goes first feeds the same exchange with send / recv_combine.  Both must get
    the attention of the whole sequence, and the same bytes as each other."""
    H, Hkv, Dh = shape
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev); gen.manual_seed(11)
    whole, parts = _split_caches(dev, 4096, H, Hkv, Dh, 2, gen)
    ranks = [D.PeerExchange(H, Dh + 2, rank=r, world=2, connect=False) for r in range(2)]
    for r in ranks:
        r.connect_local(ranks)
        r.set_wait_limit_ms(200)
    for epoch in range(4):
        q = torch.randn(1, H, Dh, device=dev, generator=gen).to(torch.bfloat16)
        want = whole.decode(0, q).float()
        first, second = (0, 1) if epoch % 2 == 0 else (1, 0)
        p_first = parts[first].decode_partial(0, q)
        ranks[first].send(p_first)
        n0 = parts[second].launch_count
        out_second = parts[second].decode_exchange(0, q, ranks[second])
        assert parts[second].launch_count - n0 == 1                  # attention + exchange + combine: one kernel
        out_first = ranks[first].recv_combine(p_first, torch.bfloat16).view(1, H, Dh)
        for r in ranks:
            r.status()
        assert torch.equal(out_first, out_second)
        torch.testing.assert_close(out_second.float(), want, rtol=2e-3, atol=1e-2)
    for c in parts + [whole]:
        c.close()
    for r in ranks:
        r.close()


def test_decode_exchange_alone_in_the_world_equals_decode():
    from titan_engine_b200 import PagedKVCache
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev); gen.manual_seed(12)
    whole, parts = _split_caches(dev, 2048, 32, 8, 128, 1, gen)
    ex = D.PeerExchange(32, 130, rank=0, world=1)
    for _ in range(3):
        q = torch.randn(1, 32, 128, device=dev, generator=gen).to(torch.bfloat16)
        assert torch.equal(whole.decode_exchange(0, q, ex), whole.decode(0, q))
    ex.status()
    ex.close(); whole.close(); parts[0].close()
