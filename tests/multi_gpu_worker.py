"""Child process of the multi-GPU tests: one rank per GPU over NCCL.  Checks the tensor-parallel
decoder layer and the expert-parallel MoE layer against the same layer computed on one GPU."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def main():
    import torch
    import torch.distributed as dist

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
        want = part.clone()
        dist.all_reduce(want)
        got = part.clone()
        comm.allreduce_(got)
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2), ("peer all-reduce", n, dt)
    ints = torch.full((2048,), float(rank + 1), device=dev, dtype=torch.float32)
    for _ in range(50):
        t2 = ints.clone()
        comm.allreduce_(t2)
        assert float(t2[0]) == world * (world + 1) / 2 and float(t2[-1]) == world * (world + 1) / 2
    ops.Context.get(rank).check()
    # the tensor-parallel layer again, now reducing through peer memory
    for m in (1, 8):
        x_a, x_o, x_m = rn(m, 512), rn(m, k_o), rn(m, 512)
        layer = parallel.TpDecoderLayer.from_full(comm, shape, w_qkv, w_o, w_gu, w_d, world, rank)
        lo, hi = parallel.tp_row_split_cols(k_o, world, rank)
        _, o, down = layer.forward(x_a, x_o[:, lo:hi].contiguous(), x_m)
        _, o_f, down_f = parallel.TpDecoderLayer(None, w_qkv, w_o, w_gu, w_d).forward(x_a, x_o, x_m)
        for got, want, what in ((o, o_f, "o"), (down, down_f, "down")):
            err = float((got.float() - want.float()).abs().max()) / float(want.float().abs().max())
            assert err < 2e-2, ("peer tp", what, m, err)

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
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok", flush=True)


if __name__ == "__main__":
    main()
