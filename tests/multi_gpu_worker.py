"""Child process of the multi-GPU tests: one rank per GPU over NCCL (2, 4 or 8 ranks).  Checks the
tensor-parallel decoder layer and the expert-parallel MoE layer against the same layer computed on one
GPU (small shapes, many calls in a row), and one Qwen3-8B-shaped tensor-parallel layer and one
Qwen3-30B-A3B-shaped expert-parallel layer against the oracle on the unsharded weights."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    import torch
    import torch.distributed as dist

    from izwi_b200 import _lib as L
    from izwi_b200 import moe, ops, parallel
    from izwi_b200.workloads import DecoderShape

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    comm = parallel.Comm(rank)
    gen = torch.Generator(device=dev).manual_seed(11)        # identical tensors on every rank
    rn = lambda *s, std=1.0: (torch.randn(*s, device=dev, generator=gen) * std).to(torch.bfloat16)  # noqa: E731

    # ---- tensor parallel ----
    shape = DecoderShape("tiny", 1, 512, 8, 4, 64, 1024)
    (_, n_qkv, _), (_, _, k_o), (_, n_gu, _), (_, _, k_d) = shape.projections
    w_qkv, w_o = rn(n_qkv, 512, std=0.03), rn(512, k_o, std=0.03)
    w_gu, w_d = rn(n_gu, 512, std=0.03), rn(512, k_d, std=0.03)
    for m in (1, 8, 200):
        x_a, x_o, x_m = rn(m, 512), rn(m, k_o), rn(m, 512)
        layer = parallel.TpDecoderLayer.from_full(comm, shape, w_qkv, w_o, w_gu, w_d, world, rank)
        lo, hi = parallel.tp_row_split_cols(k_o, world, rank)
        qkv, o, down = layer.forward(x_a, x_o[:, lo:hi].contiguous(), x_m)
        full = parallel.TpDecoderLayer(None, w_qkv, w_o, w_gu, w_d)
        qkv_f, o_f, down_f = full.forward(x_a, x_o, x_m)
        rows = torch.from_numpy(parallel.tp_qkv_rows(8, 4, 64, world, rank)).to(dev)
        assert torch.allclose(qkv.float(), qkv_f[:, rows].float(), rtol=2e-2, atol=2e-2), "tp qkv"
        for got, want, what in ((o, o_f, "o"), (down, down_f, "down")):
            err = float((got.float() - want.float()).abs().max()) / float(want.float().abs().max())
            assert err < 2e-2, (what, m, err)
    # all-reduce exactness on integers
    t = torch.full((4096,), float(rank + 1), device=dev, dtype=torch.float32)
    comm.allreduce_(t)
    assert float(t[0]) == world * (world + 1) / 2

    # ---- one-shot all-reduce over peer memory against NCCL, many calls in a row ----
    comm.enable_peer_allreduce(32 << 20)                           # one-shot up to 1 MB, two-shot above
    g2 = torch.Generator(device=dev).manual_seed(100 + rank)       # different partial sums per rank
    for n, dt in ((8, torch.bfloat16), (4096, torch.bfloat16), (131072, torch.bfloat16), (524288, torch.bfloat16),
                  (4, torch.float32), (65536, torch.float32), (524296, torch.bfloat16), (4 << 20, torch.bfloat16),
                  (16 << 20, torch.bfloat16), (1 << 20, torch.float32), ((1 << 20) + 4, torch.float32),
                  ((2 << 20) + 6, torch.bfloat16)) * 3:
        part = torch.randn(n, device=dev, generator=g2).to(dt)
        want = part.float().clone()
        dist.all_reduce(want)                                      # NCCL in fp32: the exact sum, whatever the rank count
        got = part.clone()
        comm.allreduce_(got)
        # fp32 accumulation in rank order, one rounding to the message's type: within one bf16 step of the exact sum
        assert torch.allclose(got.float(), want, rtol=8e-3 if dt == torch.bfloat16 else 1e-5, atol=1e-3), ("peer all-reduce", n, dt)
    ints = torch.full((2048,), float(rank + 1), device=dev, dtype=torch.float32)
    for _ in range(50):
        t2 = ints.clone()
        comm.allreduce_(t2)
        assert float(t2[0]) == world * (world + 1) / 2 and float(t2[-1]) == world * (world + 1) / 2
    ops.Context.get(rank).check()
    # the tensor-parallel layer again, now reducing through peer memory: decode sizes take the one-shot
    # kernel on the side stream, 2100 rows (2.1 MB per sum) the copy-free two-shot path through the
    # region, twice in a row so that both region buffers are reused
    for m in (1, 8, 2100, 2100):
        x_a, x_o, x_m = rn(m, 512), rn(m, k_o), rn(m, 512)
        layer = parallel.TpDecoderLayer.from_full(comm, shape, w_qkv, w_o, w_gu, w_d, world, rank)
        lo, hi = parallel.tp_row_split_cols(k_o, world, rank)
        _, o, down = layer.forward(x_a, x_o[:, lo:hi].contiguous(), x_m)
        comm.join()                                                # the sums ran on the side stream
        _, o_f, down_f = parallel.TpDecoderLayer(None, w_qkv, w_o, w_gu, w_d).forward(x_a, x_o, x_m)
        for got, want, what in ((o, o_f, "o"), (down, down_f, "down")):
            err = float((got.float() - want.float()).abs().max()) / float(want.float().abs().max())
            assert err < 2e-2, ("peer tp", what, m, err)

    # ---- one Qwen3-8B-shaped layer (hidden 4096, 32 / 8 heads of 128, intermediate 12288) against the
    # oracle's float64-checked products of the UNSHARDED weights on sampled token rows; the small
    # layers above are compared with the same layer on one GPU, which is a second hop ----
    sys.path.insert(0, str(ROOT / "oracle"))
    import numpy as np

    import izwi_oracle as o
    from izwi_b200.workloads import QWEN3_8B
    (_, n_qkv8, h8), (_, _, k_o8), (_, n_gu8, _), (_, _, k_d8) = QWEN3_8B.projections
    full8 = (rn(n_qkv8, h8, std=0.02), rn(h8, k_o8, std=0.02), rn(n_gu8, h8, std=0.02), rn(h8, k_d8, std=0.02))
    layer8 = parallel.TpDecoderLayer.from_full(comm, QWEN3_8B, *full8, world, rank)
    mine = parallel.tp_qkv_rows(QWEN3_8B.q_heads, QWEN3_8B.kv_heads, QWEN3_8B.head_dim, world, rank)
    lo8, hi8 = parallel.tp_row_split_cols(k_o8, world, rank)
    f32 = lambda t: t.float().cpu().numpy()  # noqa: E731
    for m in (1, 32, 2048):
        x_a, x_o, x_m = rn(m, h8), rn(m, k_o8), rn(m, h8)
        qkv, o_sum, down = layer8.forward(x_a, x_o[:, lo8:hi8].contiguous(), x_m)
        comm.join()
        torch.cuda.synchronize()
        rows = sorted({0, m // 2, m - 1})
        checks = [(qkv[rows], o.linear(f32(x_a[rows]), f32(full8[0])[mine]), "qkv"),
                  (o_sum[rows], o.linear(f32(x_o[rows]), f32(full8[1])), "o")]
        gu = o.linear(f32(x_m[rows]), f32(full8[2]))
        if m <= 32:
            gu = o.bf16_round(gu)                                    # the decode path stores gate/up in bf16
        hid = o.bf16_round(o.silu_mul(gu[:, : n_gu8 // 2], gu[:, n_gu8 // 2:]))
        checks.append((down[rows], o.linear(hid, f32(full8[3])), "down"))
        for got, want, what in checks:
            rel, cos = o.rel_err_and_cosine(f32(got), want)
            assert rel <= 2e-2 and cos >= 0.9999, ("qwen3-8b layer vs oracle", what, m, rel, cos)
    del layer8, full8
    ops.Context.get(rank).check()

    # ---- expert parallel ----
    h, inter, e, k = 512, 256, 16, 4
    wr, br = rn(e, h, std=h ** -0.5), rn(e, std=0.5)
    wgu, wd = rn(e, 2 * inter, h, std=0.03), rn(e, h, inter, std=0.03)
    lo_e, hi_e = parallel.ep_expert_range(e, world, rank)
    ep_layer = parallel.EpMoeLayer(comm, wr, br, wgu[lo_e:hi_e], wd[lo_e:hi_e], e, k)
    ref_layer = moe.MoeLayer(wr, br, wgu, wd, k)
    for t_total in (world, 64, 1000):
        x_all = rn(t_total, h)
        lo_t, hi_t = parallel.split_range(t_total, world, rank)
        y, idx, wts = ep_layer.forward(x_all[lo_t:hi_t].contiguous())
        y_ref, _, idx_ref, _ = ref_layer.forward(x_all)
        assert torch.equal(idx, idx_ref[lo_t:hi_t]), "ep routing"
        err = float((y.float() - y_ref[lo_t:hi_t].float()).abs().max()) / float(y_ref.float().abs().max())
        assert err < 2e-2, ("ep", t_total, err)
    ops.Context.get(rank).check()
    # the same layer with dispatch and return over peer memory: identical routing, same tolerance,
    # many steps in a row (sequence numbers, buffer reuse), ragged and empty shares
    comm.enable_peer_ep(e, h, 600, k)
    for step, t_total in enumerate((world, 64, 1000, world + 1, 333, 1000, 1000)):
        x_all = rn(t_total, h)
        lo_t, hi_t = parallel.split_range(t_total, world, rank)
        y, idx, wts = ep_layer.forward(x_all[lo_t:hi_t].contiguous())
        y_ref, _, idx_ref, _ = ref_layer.forward(x_all)
        assert torch.equal(idx, idx_ref[lo_t:hi_t]), "peer ep routing"
        if hi_t > lo_t:
            err = float((y.float() - y_ref[lo_t:hi_t].float()).abs().max()) / float(y_ref.float().abs().max())
            assert err < 2e-2, ("peer ep", step, t_total, err)
        ops.Context.get(rank).check()
    # ---- one Qwen3-30B-A3B-shaped layer (128 experts, hidden 2048, intermediate 768, top-8) over peer
    # memory against the oracle on the unsharded weights: routing of this rank's tokens bit-exact
    # against the oracle's top-k of the library's own logits, sampled tokens' outputs in tolerance ----
    torch.cuda.synchronize()
    dist.barrier()                       # no rank may still be storing into a buffer that is about to be freed
    L.lib().izb_ep_destroy(comm.ep)
    comm.ep = None
    h, inter, e, k = 2048, 768, 128, 8
    wr, br = rn(e, h, std=h ** -0.5), rn(e, std=0.5)
    wgu, wd = rn(e, 2 * inter, h, std=0.02), rn(e, h, inter, std=0.02)
    lo_e, hi_e = parallel.ep_expert_range(e, world, rank)
    big = parallel.EpMoeLayer(comm, wr, br, wgu[lo_e:hi_e].clone(), wd[lo_e:hi_e].clone(), e, k)
    comm.enable_peer_ep(e, h, (4096 + world - 1) // world, k)
    for t_total in (64, 4096):
        x_all = rn(t_total, h)
        lo_t, hi_t = parallel.split_range(t_total, world, rank)
        x = x_all[lo_t:hi_t].contiguous()
        y, idx, wts = big.forward(x)
        torch.cuda.synchronize()
        logits = f32(big.logits)                                    # the router logits the layer chose from
        rel, cos = o.rel_err_and_cosine(logits, o.moe_router_logits(f32(x), f32(wr), f32(br)))
        assert rel <= 2e-2 and cos >= 0.9999, ("ep router logits vs oracle", t_total, rel, cos)
        want_idx, want_w = o.moe_topk(logits, k)
        assert np.array_equal(idx.cpu().numpy(), want_idx), ("ep routing vs oracle", t_total)
        assert np.abs(f32(wts) - want_w).max() < 1e-6
        toks = sorted({0, (hi_t - lo_t) // 2, hi_t - lo_t - 1})
        want = np.zeros((len(toks), h), dtype=np.float32)
        for n, tok in enumerate(toks):
            xr = f32(x[tok:tok + 1])
            for sl in range(k):
                ex = int(want_idx[tok, sl])
                gu = o.linear(xr, f32(wgu[ex]))
                hid = o.bf16_round(o.silu_mul(gu[:, :inter], gu[:, inter:]))
                want[n] += want_w[tok, sl] * o.bf16_round(o.linear(hid, f32(wd[ex])))[0]
        rel, cos = o.rel_err_and_cosine(f32(y[toks]), want)
        assert rel <= 2e-2 and cos >= 0.9999, ("qwen3-30b-a3b layer vs oracle", t_total, rel, cos)
    ops.Context.get(rank).check()
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok", flush=True)


if __name__ == "__main__":
    main()
