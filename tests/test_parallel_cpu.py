"""Host-side sharding logic on CPU: partition arithmetic against the unsharded oracle, and the
tensor-parallel / expert-parallel exchanges among two `gloo` ranks (the data path on GPUs uses the
same plans with NCCL)."""
import os
import sys

import numpy as np
import pytest

import izwi_oracle as o
from izwi_b200 import parallel as P


def test_split_range_covers_everything():
    for n, parts in ((10, 3), (128, 8), (7, 7), (5, 8)):
        got = [P.split_range(n, parts, i) for i in range(parts)]
        assert got[0][0] == 0 and got[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
    with pytest.raises(ValueError):
        P.split_range(4, 2, 2)


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_tp_mlp_equals_unsharded(tp):
    rng = np.random.default_rng(tp)
    h, inter, m = 64, 96, 3
    x = rng.normal(size=(m, h)).astype(np.float32)
    wgu = rng.normal(0, 0.1, (2 * inter, h)).astype(np.float32)
    wd = rng.normal(0, 0.1, (h, inter)).astype(np.float32)
    want = o.mlp_forward(x, wgu, wd, inter)
    acc = np.zeros_like(want)
    for r in range(tp):
        rows = P.tp_gate_up_rows(inter, tp, r)
        lo, hi = P.tp_row_split_cols(inter, tp, r)
        acc += o.mlp_forward(x, wgu[rows], wd[:, lo:hi], hi - lo)
    assert np.abs(acc - want).max() < 1e-4


@pytest.mark.parametrize("tp", [1, 2, 4, 8, 16])
def test_tp_qkv_rows_follow_heads(tp):
    qh, kvh, hd = 32, 8, 4
    seen_q = []
    for r in range(tp):
        rows = P.tp_qkv_rows(qh, kvh, hd, tp, r)
        nq = qh // tp * hd
        seen_q.extend(rows[:nq].tolist())
        k_rows, v_rows = rows[nq: nq + (len(rows) - nq) // 2], rows[nq + (len(rows) - nq) // 2:]
        assert (v_rows - k_rows == kvh * hd).all()
        # the kv head of each local query head is present
        for q_row in rows[:nq:hd]:
            kv_head = (q_row // hd) // (qh // kvh)
            assert qh * hd + kv_head * hd in k_rows
    assert sorted(seen_q) == list(range(qh * hd))


def test_ep_plans_are_consistent():
    rng = np.random.default_rng(0)
    e, ep, k = 16, 4, 2
    all_off = []
    for r in range(ep):
        idx = np.stack([rng.choice(e, k, replace=False) for _ in range(10 + r)]).astype(np.int32)
        off, _ = o.moe_permute(idx, e)
        all_off.append(off)
    all_off = np.stack(all_off)
    send = np.stack([P.ep_send_rows(all_off[r], ep) for r in range(ep)])       # [src, dst]
    for r in range(ep):
        recv, ids = P.ep_recv_plan(all_off, ep, r)
        assert (recv == send[:, r]).all()
        assert len(ids) == recv.sum() and (ids >= 0).all() and (ids < e // ep).all()
    assert send.sum() == sum((10 + r) * k for r in range(ep))


def _ep_worker(rank, world, port, out):
    """One gloo rank of an expert-parallel MoE layer computed with the NumPy oracle."""
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)                       # same weights and tokens on every rank
    t, h, inter, e, k = 12, 16, 8, 8, 2
    x_all = rng.normal(size=(t, h)).astype(np.float32)
    wr = rng.normal(size=(e, h)).astype(np.float32)
    wg = rng.normal(0, 0.3, (e, inter, h)).astype(np.float32)
    wu = rng.normal(0, 0.3, (e, inter, h)).astype(np.float32)
    wd = rng.normal(0, 0.3, (e, h, inter)).astype(np.float32)
    want, _ = o.moe_forward(x_all, wr, None, wg, wu, wd, k, round_bf16=False)
    lo_t, hi_t = P.split_range(t, world, rank)
    x = x_all[lo_t:hi_t]
    idx, wts = o.moe_topk(o.moe_router_logits(x, wr), k)
    off, perm = o.moe_permute(idx, e)
    x_perm = x[perm // k]
    gathered = [None] * world
    dist.all_gather_object(gathered, off)
    all_off = np.stack(gathered)
    send_rows = P.ep_send_rows(off, world)
    recv_rows, ids = P.ep_recv_plan(all_off, world, rank)
    # dispatch
    cuts = np.concatenate([[0], np.cumsum(send_rows)])
    blocks = [None] * world
    dist.all_gather_object(blocks, [x_perm[cuts[d]:cuts[d + 1]] for d in range(world)])
    recv = np.concatenate([blocks[s][rank] for s in range(world)]) if recv_rows.sum() else np.zeros((0, h), np.float32)
    assert recv.shape[0] == recv_rows.sum()
    e_lo, _ = P.ep_expert_range(e, world, rank)
    y_recv = np.zeros_like(recv)
    for row, le in enumerate(ids):
        y_recv[row] = o.moe_expert_ffn(recv[row:row + 1], wg[e_lo + le], wu[e_lo + le], wd[e_lo + le], round_bf16=False)[0]
    # return
    rc = np.concatenate([[0], np.cumsum(recv_rows)])
    blocks = [None] * world
    dist.all_gather_object(blocks, [y_recv[rc[s]:rc[s + 1]] for s in range(world)])
    y_perm = np.concatenate([blocks[d][rank] for d in range(world)])
    inv = np.empty(len(perm), np.int64)
    inv[perm] = np.arange(len(perm))
    y = np.zeros((hi_t - lo_t, h), np.float32)
    for s in range(k):
        y += wts[:, s:s + 1] * y_perm[inv[np.arange(hi_t - lo_t) * k + s]]
    err = float(np.abs(y - want[lo_t:hi_t]).max())
    # tensor-parallel all-reduce of a row-split projection
    w = rng.normal(size=(6, h)).astype(np.float32)
    clo, chi = P.tp_row_split_cols(h, world, rank)
    part = torch.from_numpy(o.linear(x_all[:, clo:chi], w[:, clo:chi]))
    dist.all_reduce(part)
    err_tp = float(np.abs(part.numpy() - o.linear(x_all, w)).max())
    out.put((rank, err, err_tp))
    dist.destroy_process_group()


def test_two_gloo_ranks_ep_and_tp():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, err_tp in results:
        assert err < 1e-4, (rank, err)
        assert err_tp < 1e-4, (rank, err_tp)


@pytest.mark.parametrize("world,e", [(2, 16), (4, 16), (8, 128), (8, 8)])
def test_peer_ep_tables_route_every_row_to_its_expert_and_home(world, e):
    """Simulates the peer-memory dispatch and return with the placement tables on random routing,
    hot experts and empty (expert, source) groups included: every row lands in a slot of its own on
    the rank that owns its expert, inside that expert's segment, in (source, order) sequence, and the
    return puts it back on the row it left from."""
    rng = np.random.default_rng(world * 100 + e)
    per = e // world
    p = rng.dirichlet(np.full(e, 0.3))
    counts = np.stack([rng.multinomial(int(rng.integers(0, 300)), p) for _ in range(world)])  # [source, expert]
    counts[:, rng.integers(0, e)] = 0                                                      # an expert nobody chose
    tabs = [P.ep_peer_tables(counts, r) for r in range(world)]
    # source rows: expert-major, tagged (source, expert, order)
    recv = [np.full((tabs[r]["total"], 3), -1, dtype=np.int64) for r in range(world)]
    for s in range(world):
        for ex in range(e):
            owner = ex // per
            for j in range(counts[s, ex]):
                slot = tabs[s]["dst_row"][ex] + j
                assert (recv[owner][slot] == -1).all(), "two rows stored to one slot"
                recv[owner][slot] = (s, ex, j)
    home = [np.full(counts[s].sum(), -1, dtype=np.int64) for s in range(world)]
    for r in range(world):
        assert (recv[r] >= 0).all(), "a received slot was never written"
        seg = tabs[r]["seg"]
        assert seg[0] == 0 and seg[-1] == counts[:, r * per:(r + 1) * per].sum()
        for l in range(per):
            rows = recv[r][seg[l]:seg[l + 1]]
            assert (rows[:, 1] == r * per + l).all()                                       # only this expert's rows
            key = rows[:, 0] * 10 ** 6 + rows[:, 2]
            assert (np.diff(key) > 0).all()                                               # source-major, in source order
            for s in range(world):
                a = tabs[r]["recv_start"][l, s]
                assert (recv[r][a:a + counts[s, r * per + l], 0] == s).all()
        # return: row i of (local expert l, source s, order j) goes home to ret_start[s, l] + j
        for i, (s, ex, j) in enumerate(recv[r]):
            slot = tabs[r]["ret_start"][s, ex - r * per] + j
            assert home[s][slot] == -1
            home[s][slot] = ex
    for s in range(world):
        assert np.array_equal(home[s], np.repeat(np.arange(e), counts[s]))                # its own expert-major order
    # consistent with the host planner of the NCCL path
    for r in range(world):
        offs = np.concatenate([np.zeros((world, 1), dtype=np.int64), np.cumsum(counts, axis=1)], axis=1)
        recv_rows, _ = P.ep_recv_plan(offs, world, r)
        assert recv_rows.sum() == tabs[r]["total"]
